"""
tcgen05 GEMM against an fp32 torch matmul, all four operand layouts, edge sizes, epilogues, and the linear autograd path.
"""

import pytest
import torch

gpu = pytest.mark.gpu


def _mk(rows, cols, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(rows, cols, device="cuda", generator=g) * 0.5).to(torch.bfloat16)


@gpu
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 384, 512), (200, 136, 72), (6700, 2048, 512), (33, 10008, 512), (1, 8, 8)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (False, False), (True, True), (True, False)])
def test_gemm_layouts(m, n, k, a_mn, b_mn):
    from returnn_b200.ops import gemm

    a_log = _mk(m, k, 1)  # logical A [m, k]
    b_log = _mk(k, n, 2)  # logical B [k, n]
    a = a_log.t().contiguous() if a_mn else a_log  # stored [k, m] or [m, k]
    b = b_log if b_mn else b_log.t().contiguous()  # stored [k, n] or [n, k]
    if (a.stride(0) % 8) or (b.stride(0) % 8):
        pytest.skip("pitch not a multiple of 8 elements")
    out = gemm.gemm(a, b, m=m, n=n, k=k, a_mn_major=a_mn, b_mn_major=b_mn)
    gemm.check_status()
    ref = a_log.float() @ b_log.float()
    torch.testing.assert_close(out.float(), ref, atol=0.06 + 2e-3 * k ** 0.5, rtol=2e-2)


@gpu
@pytest.mark.parametrize("act", [None, "relu", "silu", "gelu"])
def test_gemm_epilogue(act):
    from returnn_b200.ops import gemm

    m, n, k = 300, 264, 136
    a, b = _mk(m, k, 3), _mk(k, n, 4)
    bias = torch.randn(n, device="cuda")
    z, y = gemm.gemm(a, b, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, bias=bias, act=act, want_act_output=True)
    gemm.check_status()
    zr = a.float() @ b.float() + bias
    fn = {None: lambda t: t, "relu": torch.relu, "silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu}[act]
    torch.testing.assert_close(z.float(), zr, atol=0.08, rtol=2e-2)
    torch.testing.assert_close(y.float(), fn(zr), atol=0.08, rtol=2e-2)
    out32 = torch.ones(m, n, device="cuda")
    gemm.gemm(a, b, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, out=out32, accumulate=True, alpha=0.5)
    torch.testing.assert_close(out32, 1.0 + 0.5 * (a.float() @ b.float()), atol=0.05, rtol=1e-2)


@gpu
def test_linear_autograd_matches_fp32():
    from returnn_b200.ops import gemm, linear

    torch.manual_seed(0)
    x = (torch.randn(5, 77, 512, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(512, 2048, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(2048, device="cuda").to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(5, 77, 2048, device="cuda").to(torch.bfloat16)
    assert gemm.ENABLED
    y = linear.linear(x, w, b, "silu")
    y.backward(dy)
    gemm.check_status()
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.silu(xr @ wr + br)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, atol=0.05, rtol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=0.05, rtol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=0.4, rtol=3e-2)
    torch.testing.assert_close(b.grad.float(), br.grad, atol=0.5, rtol=3e-2)


@gpu
@pytest.mark.parametrize("m,n,k", [(300, 264, 136), (1000, 512, 2048), (77, 72, 64)])
def test_gemm_fused_epilogue_resid_dropout(m, n, k):
    """out = resid + 0.5 * dropout(a·b + bias), mask identical to the stand-alone dropout kernel at the same offset"""
    from returnn_b200.ops import gemm, elementwise

    a, b = _mk(m, k, 5), _mk(k, n, 6)
    bias = torch.randn(n, device="cuda")
    resid = _mk(m, n, 7)
    seed = torch.tensor([1234, 4096], dtype=torch.int64, device="cuda")
    off = seed[1:2].clone()
    site = 8 * 1000
    out = gemm.gemm(a, b, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, bias=bias, dropout_p=0.25, dropout_seed=seed[0:1],
                    dropout_offset=off, dropout_site=site, resid=resid, res_scale=0.5)
    gemm.check_status()
    y = (a.float() @ b.float() + bias)
    # the mask of the stand-alone kernel with the same key and counter base
    ones = torch.ones(m, n, device="cuda", dtype=torch.bfloat16)
    mask = elementwise.dropout_with_state(ones, 0.25, seed[0:1], off + site).float()
    ref = resid.float() + 0.5 * y * mask
    torch.testing.assert_close(out.float(), ref, atol=0.1, rtol=2e-2)
    assert 0.6 < float((mask > 0).float().mean()) < 0.9


@gpu
@pytest.mark.parametrize("act", ["relu", "silu", "gelu"])
def test_gemm_fused_act_grad(act):
    from returnn_b200.ops import gemm

    m, n, k = 520, 2048, 512
    dy, w = _mk(m, k, 8), _mk(n, k, 9)  # dA[m,n] = dY[m,k] · W[n,k]^T
    z = _mk(m, n, 10)
    out = gemm.gemm(dy, w, m=m, n=n, k=k, a_mn_major=False, b_mn_major=False, act=act, dact_z=z)
    gemm.check_status()
    zz = z.float().requires_grad_(True)
    fn = {"relu": torch.relu, "silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu}[act]
    da = dy.float() @ w.float().t()
    (g,) = torch.autograd.grad(fn(zz), zz, da)
    torch.testing.assert_close(out.float(), g, atol=0.15, rtol=3e-2)


@gpu
@pytest.mark.parametrize("m,n,k", [(512, 2048, 6700), (512, 512, 6656), (136, 72, 1000), (512, 10240, 3000)])
def test_gemm_split_k_atomic(m, n, k):
    """weight-gradient form dW += X^T·dY with the contraction split over CTAs"""
    from returnn_b200.ops import gemm

    x, dy = _mk(k, m, 11), _mk(k, n, 12)
    acc = torch.full((m, n), 2.0, device="cuda")
    gemm.gemm(x, dy, m=m, n=n, k=k, a_mn_major=True, b_mn_major=True, out=acc, atomic=True)
    gemm.gemm(x, dy, m=m, n=n, k=k, a_mn_major=True, b_mn_major=True, out=acc, atomic=True, split_k=3)
    gemm.check_status()
    ref = 2.0 + 2.0 * (x.float().t() @ dy.float())
    torch.testing.assert_close(acc, ref, atol=0.05 * k ** 0.5, rtol=2e-2)


@pytest.mark.gpu
def test_linear_arena_padded_out():
    """output layer of width 1001 (not a multiple of 8) through the 8-aligned computation: loss and gradients as torch in fp32"""
    from returnn_b200.ops import gemm as G
    from returnn_b200.parallel.arena import ParamArena

    torch.manual_seed(3)
    dev = torch.device("cuda")
    m, k, n = 700, 256, 1001
    lin = torch.nn.Module()
    lin.weight = torch.nn.Parameter(torch.randn(k, n, device=dev) * 0.05)
    lin.bias = torch.nn.Parameter(torch.randn(n, device=dev) * 0.1)
    arena = ParamArena(list(lin.named_parameters()))
    arena.zero_grad()
    x = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    tgt = torch.randint(0, n, (m,), device=dev)
    y = G.linear_arena_padded_out(x, lin.weight, lin.bias, arena)
    assert y is not None and y.shape == (m, 1008)
    logp = torch.log_softmax(y.float(), dim=-1)
    assert float(logp[:, n:].exp().max()) == 0.0
    loss = -logp.gather(1, tgt[:, None]).sum()
    loss.backward()
    # fp32 reference on the bf16-rounded operands
    xr = x.detach().float().requires_grad_(True)
    wr = lin.weight.detach().to(torch.bfloat16).float().requires_grad_(True)
    br = lin.bias.detach().clone().requires_grad_(True)
    yr = xr @ wr + br
    loss_r = -torch.log_softmax(yr, dim=-1).gather(1, tgt[:, None]).sum()
    loss_r.backward()
    assert abs(float(loss) - float(loss_r)) / abs(float(loss_r)) < 2e-3
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=2e-2, rtol=5e-2)
    by_name = {s.name: s for s in arena.slots}
    for name, ref in (("weight", wr.grad), ("bias", br.grad)):
        s = by_name[name]
        got = arena.flat_grad[s.offset: s.offset + s.numel].view(ref.shape)
        torch.testing.assert_close(got, ref, atol=3e-2, rtol=5e-2)
