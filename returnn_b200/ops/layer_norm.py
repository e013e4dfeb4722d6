"""
LayerNorm / RMSNorm over the last axis, one pass per row.

Native path (CUDA, bf16 or fp32 rows): one warp-group per row; mean/rstd saved for backward; the backward kernel
produces dx and per-CTA partial sums of dgamma/dbeta which a second small kernel reduces (scratch memory).
"""

from __future__ import annotations
from typing import Optional
import ctypes
import torch
from . import _lib

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        rows, n = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        fn = _lib.bind("rb200_layer_norm_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _i32, _i32, _vp])
        g = gamma.contiguous()
        b = beta.contiguous() if beta is not None else None
        _lib.check(fn(_p(x2), _p(g), _p(b), _p(y), _p(mean), _p(rstd), rows, n, eps, 1 if x2.dtype == torch.bfloat16 else 0,
                      1 if g.dtype == torch.bfloat16 else 0, 1 if rms else 0, _lib.stream_ptr()), "layer_norm_fwd")
        _lib.count_launch()
        ctx.save_for_backward(x2, g, mean, rstd)
        ctx.has_beta = beta is not None
        ctx.rms = rms
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, g, mean, rstd = ctx.saved_tensors
        rows, n = x2.shape
        dy2 = dy.reshape(rows, n).contiguous()
        dx = torch.empty_like(x2)
        n_part = min(296, max(1, (rows + 31) // 32))
        bf16_x = x2.dtype == torch.bfloat16
        if bf16_x and n <= 512 and rows > 0 and dy2.dtype == torch.bfloat16:
            # one kernel: the column sums are added onto zeroed dgamma / dbeta inside the row pass (the form the native encoder uses)
            sums = torch.zeros(2, n, dtype=torch.float32, device=x2.device)
            dgamma, dbeta = sums[0], sums[1]
            fn = _lib.bind("rb200_layer_norm_bwd_ex", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp])
            _lib.check(fn(_p(x2), _p(dy2), _p(g), _p(mean), _p(rstd), _p(dx), None, _p(dgamma), _p(dbeta), rows, n, n_part, 1,
                          1 if g.dtype == torch.bfloat16 else 0, 1 if ctx.rms else 0, None, 1, _lib.stream_ptr()), "layer_norm_bwd")
            _lib.count_launch()
        else:
            part = torch.empty(2, n_part, n, dtype=torch.float32, device=x2.device)
            dgamma = torch.empty(n, dtype=torch.float32, device=x2.device)
            dbeta = torch.empty(n, dtype=torch.float32, device=x2.device)
            fn = _lib.bind("rb200_layer_norm_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp])
            _lib.check(fn(_p(x2), _p(dy2), _p(g), _p(mean), _p(rstd), _p(dx), _p(part), _p(dgamma), _p(dbeta), rows, n, n_part,
                          1 if bf16_x else 0, 1 if g.dtype == torch.bfloat16 else 0, 1 if ctx.rms else 0,
                          _lib.stream_ptr()), "layer_norm_bwd")
            _lib.count_launch(2)
        return dx.reshape(ctx.shape), dgamma.to(g.dtype), (dbeta.to(g.dtype) if ctx.has_beta else None), None, None


def _native_ok(x: torch.Tensor, gamma: torch.Tensor) -> bool:
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32):
        return False
    n = x.shape[-1]
    if n % 8 != 0 or n > 2048:  # the backward kernel keeps a row in registers
        return False
    return _lib.use_native(x, gamma)


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """(x - mean) * rsqrt(var + eps) * gamma + beta over the last axis"""
    if _native_ok(x, gamma):
        return _LayerNormFn.apply(x, gamma, beta, float(eps), False)
    return layer_norm_reference(x, gamma, beta, eps)


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * gamma (+ beta)"""
    if _native_ok(x, gamma):
        return _LayerNormFn.apply(x, gamma, beta, float(eps), True)
    return rms_norm_reference(x, gamma, beta, eps)


def layer_norm_reference(x, gamma, beta, eps):
    """plain torch, statistics in fp32"""
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = (xf - mean).square().mean(dim=-1, keepdim=True)
    y = (xf - mean) * torch.rsqrt(var + eps) * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(x.dtype)


def rms_norm_reference(x, gamma, beta, eps):
    """plain torch, statistics in fp32"""
    xf = x.float()
    y = xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps) * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(x.dtype)
