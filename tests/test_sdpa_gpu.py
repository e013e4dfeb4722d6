"""scaled-dot-product attention kernels against plain PyTorch fp32"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, H, D, Tq, Tk, causal, with_lens, seed=0):
    from returnn_b200.ops import sdpa as S

    torch.manual_seed(seed)
    dev = torch.device("cuda")
    bf = torch.bfloat16
    q = (torch.randn(B, Tq, H * D, device=dev) * 0.7).to(bf).requires_grad_(True)
    k = (torch.randn(B, Tk, H * D, device=dev) * 0.7).to(bf).requires_grad_(True)
    v = (torch.randn(B, Tk, H * D, device=dev) * 0.7).to(bf).requires_grad_(True)
    lens = torch.randint(max(1, Tk // 2), Tk + 1, (B,), device=dev, dtype=torch.int32) if with_lens else None
    assert S.supports(q, k, H)
    out = S.sdpa(q, k, v, num_heads=H, k_lens=lens, causal=causal)
    w = torch.randn_like(out, dtype=torch.float32)
    (out.float() * w).sum().backward()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = S.sdpa_reference(qr, kr, vr, num_heads=H, k_lens=lens, causal=causal)
    (ref * w).sum().backward()
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    for got, want, name in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk"), (v.grad, vr.grad, "dv")):
        err = (got.float() - want).abs().max().item()
        scale = want.abs().max().item() + 1e-6
        assert err / scale < 3e-2, (name, err, scale)


@pytest.mark.parametrize("B,H,D,Tq,Tk,causal,with_lens", [
    (3, 2, 64, 70, 70, False, True),     # encoder self attention with padding
    (2, 4, 64, 33, 33, True, False),     # causal decoder self attention
    (2, 2, 64, 17, 130, False, True),    # cross attention: short queries, long padded keys
    (1, 1, 128, 1, 65, True, False),     # one decoding step against a cache (the query is the last position)
    (2, 8, 64, 128, 192, False, False),  # sizes on tile boundaries
    (2, 2, 64, 40, 300, False, True),    # key rows of two register chunks per lane
    (1, 2, 64, 64, 600, False, True),    # ... and of four
    (2, 2, 64, 200, 200, True, True),    # causal with padding, a whole warp per row
])
def test_sdpa_matches_reference(B, H, D, Tq, Tk, causal, with_lens):
    _case(B, H, D, Tq, Tk, causal, with_lens)


def test_sdpa_dropout_statistics_and_4d_entry():
    from returnn_b200.ops import sdpa as S, attention as A

    torch.manual_seed(1)
    dev = torch.device("cuda")
    B, H, D, T = 2, 2, 64, 96
    q = torch.randn(B, T, H * D, device=dev).to(torch.bfloat16)
    k = torch.randn(B, T, H * D, device=dev).to(torch.bfloat16)
    v = torch.ones(B, T, H * D, device=dev).to(torch.bfloat16)
    # with constant values the output is the kept probability mass / (1-p): mean 1, and not identically 1
    out = S.sdpa(q, k, v, num_heads=H, dropout_p=0.5).float()
    assert abs(out.mean().item() - 1.0) < 0.05 and out.std().item() > 0.01
    # the [B, H, T, D] entry used by rf.dot_attention
    q4 = q.view(B, T, H, D).transpose(1, 2)
    k4 = k.view(B, T, H, D).transpose(1, 2)
    vv = torch.randn(B, T, H * D, device=dev).to(torch.bfloat16)
    v4 = vv.view(B, T, H, D).transpose(1, 2)
    lens = torch.tensor([96, 50], device=dev, dtype=torch.int32)
    got = A.sdpa(q4, k4, v4, kv_lens=lens, scale=D ** -0.5, causal=False)
    want = A.sdpa_reference(q4.float(), k4.float(), v4.float(), kv_lens=lens, scale=D ** -0.5, causal=False)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("layout", ["per_head_interleaved", "three_blocks"])
def test_sdpa_heads_reads_slices_of_a_fused_projection_in_place(layout):
    """q / k / v as strided views of one [B, T, 3 * H * D] tensor (both common column orders): same result and gradients as on copies"""
    from returnn_b200.ops import sdpa as S

    torch.manual_seed(3)
    dev = torch.device("cuda")
    B, T, H, D = 3, 75, 4, 64
    qkv = (torch.randn(B, T, 3 * H * D, device=dev) * 0.7).to(torch.bfloat16).requires_grad_(True)
    lens = torch.tensor([75, 40, 9], device=dev, dtype=torch.int32)

    def split(x):
        if layout == "per_head_interleaved":  # [.., H, 3 * D] -> three [.., H, D] slices
            x4 = x.view(B, T, H, 3 * D)
            return x4[..., :D], x4[..., D: 2 * D], x4[..., 2 * D:]
        x4 = x.view(B, T, 3, H, D)
        return x4[:, :, 0], x4[:, :, 1], x4[:, :, 2]

    q, k, v = split(qkv)
    assert not q.is_contiguous() and S._rows(q)[0].data_ptr() == q.data_ptr()  # addressed in place
    w = torch.randn(B, T, H, D, device=dev)
    out = S.sdpa_heads(q, k, v, k_lens=lens)
    (out.float() * w).sum().backward()
    got = qkv.grad.clone()
    qkv.grad = None
    qc, kc, vc = (t.contiguous().view(B, T, H * D) for t in split(qkv))
    ref = S.sdpa_reference(qc, kc, vc, num_heads=H, k_lens=lens).view(B, T, H, D)
    (ref * w).sum().backward()
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    scale = float(qkv.grad.abs().max())
    assert float((got.float() - qkv.grad.float()).abs().max()) / scale < 3e-2
