"""
The central kernels as registered PyTorch operators (``torch.ops.returnn_b200.*``): schema, CUDA implementation (the entry points of
``librb200.so``), CPU implementation (plain torch, for tests), fake / meta implementation (shapes and dtypes without running a
kernel) and autograd formula. With that they work under fake-tensor tracing, ``torch.export``, ``torch.library.opcheck`` and inside
user code that is itself traced, where a bare ``ctypes`` call on data pointers cannot.

    y = torch.ops.returnn_b200.gemm(a, b, trans_a, trans_b)            # bf16 [m, k] x [k, n] -> bf16 [m, n] on the tcgen05 GEMM
    y = torch.ops.returnn_b200.linear(x, weight, bias, activation)      # x[..., in] @ weight[in, out] (+ bias) (activation)
    y, mean, rstd = torch.ops.returnn_b200.layer_norm(x, gamma, beta, eps)

The wrappers of :mod:`returnn_b200.ops` remain the way the framework itself calls the kernels (they fuse more: arena gradients,
dropout, residuals); these operators are the interoperable surface. The reference reaches its native ops from torch through a
``torch.autograd.Function`` over a compiled module (returnn/torch/util/native_op.py:17-140, native_op_code_compiler.py).
"""

from __future__ import annotations
from typing import Optional, Tuple
import torch
from torch.library import custom_op

__all__ = ["gemm", "linear", "layer_norm"]

_ACTS = ("", "relu", "silu", "gelu")


def _native(t: torch.Tensor) -> bool:
    from . import gemm as _gemm

    return t.is_cuda and _gemm.available(t)


# ---------------------------------------------------------------------------------------------------------------------------------
@custom_op("returnn_b200::gemm", mutates_args=())
def gemm(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False) -> torch.Tensor:
    """``op(a) @ op(b)`` for 2-D bf16 operands, fp32 accumulation, bf16 result"""
    m, k = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    n = b.shape[0] if trans_b else b.shape[1]
    if _native(a) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and all(v % 8 == 0 for v in (a.shape[1], b.shape[1], n)):
        from . import gemm as _gemm

        a_, b_ = a.contiguous(), b.contiguous()
        # the kernel's operand descriptions: A stored [m][k] or [k][m]; B stored [n][k] or [k][n]
        return _gemm.gemm(a_, b_, m=m, n=n, k=k, a_mn_major=trans_a, b_mn_major=not trans_b)
    aa = a.t() if trans_a else a
    bb = b.t() if trans_b else b
    return (aa.float() @ bb.float()).to(a.dtype)


@gemm.register_fake
def _(a, b, trans_a=False, trans_b=False):
    m = a.shape[1] if trans_a else a.shape[0]
    n = b.shape[0] if trans_b else b.shape[1]
    return a.new_empty((m, n))


def _gemm_setup(ctx, inputs, output):
    a, b, ta, tb = inputs
    ctx.save_for_backward(a, b)
    ctx.ta, ctx.tb = ta, tb


def _gemm_backward(ctx, dy):
    a, b = ctx.saved_tensors
    ta, tb = ctx.ta, ctx.tb
    dy = dy.contiguous()
    # C = op(A) op(B):  d op(A) = dC op(B)^T,  d op(B) = op(A)^T dC; the transposes of the stored operands are flags of the same op
    if not ta:
        da = gemm(dy, b, False, not tb)
    else:
        da = gemm(b, dy, tb, True)
    if not tb:
        db = gemm(a, dy, not ta, False)
    else:
        db = gemm(dy, a, True, ta)
    return da, db, None, None


gemm.register_autograd(_gemm_backward, setup_context=_gemm_setup)


# ---------------------------------------------------------------------------------------------------------------------------------
@custom_op("returnn_b200::linear", mutates_args=())
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, activation: str = "") -> torch.Tensor:
    """``act(x[..., in] @ weight[in, out] + bias)``; ``activation`` one of "", "relu", "silu", "gelu" (fused into the GEMM epilogue)"""
    assert activation in _ACTS, "activation %r not in %r" % (activation, _ACTS)
    from . import linear as _linear

    with torch.no_grad():
        return _linear.linear(x, weight, bias, activation or None)


@linear.register_fake
def _(x, weight, bias=None, activation=""):
    return x.new_empty(tuple(x.shape[:-1]) + (weight.shape[1],))


def _linear_setup(ctx, inputs, output):
    x, weight, bias, activation = inputs
    ctx.save_for_backward(x, weight, bias if bias is not None else x.new_empty(0), output)
    ctx.has_bias = bias is not None
    ctx.activation = activation


def _linear_backward(ctx, dy):
    x, weight, bias, y = ctx.saved_tensors
    act = ctx.activation
    dz = dy
    if act == "relu":
        dz = dy * (y > 0).to(dy.dtype)
    elif act in ("silu", "gelu"):  # needs the pre-activation: recompute it (one more GEMM; the framework's own wrappers keep it instead)
        z = linear(x, weight, bias if ctx.has_bias else None, "").float()
        if act == "silu":
            s = torch.sigmoid(z)
            dz = (dy.float() * (s * (1 + z * (1 - s)))).to(dy.dtype)
        else:
            cdf = 0.5 * (1 + torch.erf(z * 0.7071067811865476))
            pdf = torch.exp(-0.5 * z * z) * 0.3989422804014327
            dz = (dy.float() * (cdf + z * pdf)).to(dy.dtype)
    x2 = x.reshape(-1, x.shape[-1])
    dz2 = dz.reshape(-1, dz.shape[-1])
    if x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and dz2.dtype == torch.bfloat16:
        dx = gemm(dz2.contiguous(), weight, False, True)
        dw = gemm(x2.contiguous(), dz2.contiguous(), True, False)
    else:
        dx = (dz2.float() @ weight.float().t()).to(x.dtype)
        dw = (x2.float().t() @ dz2.float()).to(weight.dtype)
    db = dz2.float().sum(0).to(bias.dtype) if ctx.has_bias else None
    return dx.reshape(x.shape), dw, db, None


linear.register_autograd(_linear_backward, setup_context=_linear_setup)


# ---------------------------------------------------------------------------------------------------------------------------------
@custom_op("returnn_b200::layer_norm", mutates_args=())
def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """layer norm over the last axis; returns (y, mean [rows], rstd [rows])"""
    n = x.shape[-1]
    x2 = x.reshape(-1, n)
    xf = x2.float()
    mean = xf.mean(-1)
    rstd = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
    from . import layer_norm as _ln

    if _ln._native_ok(x, gamma):
        y = _ln.layer_norm(x.detach(), gamma.detach(), beta.detach() if beta is not None else None, eps)
    else:
        y = ((xf - mean[:, None]) * rstd[:, None] * gamma.float() + (beta.float() if beta is not None else 0.0)).to(x.dtype).reshape(x.shape)
    return y, mean, rstd


@layer_norm.register_fake
def _(x, gamma, beta, eps):
    rows = x.numel() // max(x.shape[-1], 1)
    return torch.empty_like(x), x.new_empty((rows,), dtype=torch.float32), x.new_empty((rows,), dtype=torch.float32)


def _ln_setup(ctx, inputs, output):
    x, gamma, beta, eps = inputs
    _, mean, rstd = output
    ctx.save_for_backward(x, gamma, mean, rstd)
    ctx.has_beta = beta is not None


def _ln_backward(ctx, dy, _dmean, _drstd):
    x, gamma, mean, rstd = ctx.saved_tensors
    n = x.shape[-1]
    xh = (x.reshape(-1, n).float() - mean[:, None]) * rstd[:, None]
    dyf = dy.reshape(-1, n).float()
    g = dyf * gamma.float()
    dx = (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True)) * rstd[:, None]
    dgamma = (dyf * xh).sum(0).to(gamma.dtype)
    dbeta = dyf.sum(0).to(gamma.dtype) if ctx.has_beta else None
    return dx.to(x.dtype).reshape(x.shape), dgamma, dbeta, None


layer_norm.register_autograd(_ln_backward, setup_context=_ln_setup)
