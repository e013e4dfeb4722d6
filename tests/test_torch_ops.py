"""
Registered operators (returnn_b200/ops/torch_ops.py): fake implementations give the right shapes without running anything, autograd
formulas agree with torch, and ``torch.library.opcheck`` accepts schema, fake kernel and autograd registration (CPU here, CUDA in the gpu test).
"""

import pytest
import torch

gpu = pytest.mark.gpu


def _check_values(dev, dtype, atol):
    import returnn_b200.ops.torch_ops  # noqa: F401  (registers the ops)

    torch.manual_seed(0)
    ops = torch.ops.returnn_b200
    a = torch.randn(32, 16, device=dev, dtype=dtype, requires_grad=True)
    b = torch.randn(16, 24, device=dev, dtype=dtype, requires_grad=True)
    for ta, tb in ((False, False), (True, False), (False, True), (True, True)):
        aa = a.t().contiguous().detach().requires_grad_(True) if ta else a.detach().requires_grad_(True)
        bb = b.t().contiguous().detach().requires_grad_(True) if tb else b.detach().requires_grad_(True)
        y = ops.gemm(aa, bb, ta, tb)
        ref = (aa.t() if ta else aa).float() @ (bb.t() if tb else bb).float()
        torch.testing.assert_close(y.float(), ref, atol=atol, rtol=atol)
        gy = torch.randn_like(y)
        y.backward(gy)
        ga, gb = torch.autograd.grad(ref, [aa, bb], gy.float())
        torch.testing.assert_close(aa.grad.float(), ga.float(), atol=atol * 4, rtol=atol * 4)
        torch.testing.assert_close(bb.grad.float(), gb.float(), atol=atol * 4, rtol=atol * 4)
    x = torch.randn(3, 5, 16, device=dev, dtype=dtype, requires_grad=True)
    w = (torch.randn(16, 24, device=dev, dtype=dtype) * 0.3).requires_grad_(True)
    bias = torch.randn(24, device=dev, dtype=dtype, requires_grad=True)
    for act, fn in (("", lambda z: z), ("relu", torch.relu), ("silu", torch.nn.functional.silu), ("gelu", torch.nn.functional.gelu)):
        for t in (x, w, bias):
            t.grad = None
        y = ops.linear(x, w, bias, act)
        gy = torch.randn_like(y)
        y.backward(gy)
        got = [t.grad.float().clone() for t in (x, w, bias)]
        xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, bias))
        ref = fn(xr @ wr + br)
        ref.backward(gy.float())
        torch.testing.assert_close(y.float(), ref.detach(), atol=atol * 2, rtol=atol * 2)
        for g, r in zip(got, (xr, wr, br)):
            torch.testing.assert_close(g, r.grad, atol=atol * 8, rtol=atol * 8)
    gamma = torch.rand(16, device=dev, requires_grad=True)
    beta = torch.randn(16, device=dev, requires_grad=True)
    xl = torch.randn(7, 16, device=dev, requires_grad=True)
    y, mean, rstd = ops.layer_norm(xl, gamma, beta, 1e-5)
    gy = torch.randn_like(y)
    y.backward(gy)
    got = [t.grad.clone() for t in (xl, gamma, beta)]
    xr, gr, br = (t.detach().clone().requires_grad_(True) for t in (xl, gamma, beta))
    ref = torch.nn.functional.layer_norm(xr, (16,), gr, br, 1e-5)
    ref.backward(gy)
    torch.testing.assert_close(y, ref.detach(), atol=1e-4, rtol=1e-4)
    for g, r in zip(got, (xr, gr, br)):
        torch.testing.assert_close(g, r.grad, atol=2e-4, rtol=2e-4)


def test_registered_ops_values_and_gradients_cpu():
    _check_values("cpu", torch.float32, 1e-5)


def test_registered_ops_fake_tensors_and_opcheck_cpu():
    import returnn_b200.ops.torch_ops  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode

    ops = torch.ops.returnn_b200
    with FakeTensorMode():
        a = torch.empty(64, 32, dtype=torch.bfloat16)
        b = torch.empty(48, 32, dtype=torch.bfloat16)
        assert tuple(ops.gemm(a, b, False, True).shape) == (64, 48)
        x = torch.empty(2, 9, 32)
        y = ops.linear(x, torch.empty(32, 40), torch.empty(40), "silu")
        assert tuple(y.shape) == (2, 9, 40) and y.dtype == torch.float32
        y, mean, rstd = ops.layer_norm(x, torch.empty(32), None, 1e-6)
        assert tuple(y.shape) == (2, 9, 32) and tuple(mean.shape) == (18,) and rstd.dtype == torch.float32
    a = torch.randn(8, 16, requires_grad=True)
    b = torch.randn(16, 8, requires_grad=True)
    torch.library.opcheck(ops.gemm.default, (a, b, False, False))
    torch.library.opcheck(ops.linear.default, (torch.randn(4, 16, requires_grad=True), torch.randn(16, 8, requires_grad=True), torch.randn(8, requires_grad=True), "relu"))
    torch.library.opcheck(ops.layer_norm.default, (torch.randn(4, 16, requires_grad=True), torch.rand(16, requires_grad=True), torch.randn(16, requires_grad=True), 1e-5))


@gpu
def test_registered_ops_run_the_native_kernels():
    from returnn_b200.ops import _lib

    before = _lib.launch_count()
    _check_values("cuda", torch.bfloat16, 3e-2)
    assert _lib.launch_count() > before  # the CUDA implementations went through the library, not through a torch fallback
