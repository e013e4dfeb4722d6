"""
Bindings of the optimizer kernels (``csrc/optim.cu``): fused AdamW over a flat arena, sum of squares with
per-CTA partials, Lion update.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import torch
from . import _lib

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def available() -> bool:
    """library present with the AdamW kernel"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_adamw_arena")


def lion_available(p) -> bool:
    """library present with the Lion kernel and fp32 parameter"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_lion") and p.dtype == torch.float32 and p.is_contiguous()


def sum_squares(x: torch.Tensor, scratch: torch.Tensor) -> torch.Tensor:
    """sum(x^2) as fp32 device scalar; ``scratch`` holds the per-CTA partials (>= 1025 floats)"""
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    fn = _lib.bind("rb200_sum_squares", [_vp, _i64, _i32, _vp, _vp, _vp])
    _lib.check(fn(x.data_ptr(), x.numel(), {torch.float32: 0, torch.bfloat16: 1}[x.dtype], scratch.data_ptr(), out.data_ptr(), _lib.stream_ptr()), "sum_squares")
    _lib.count_launch(2)
    return out[0]


def adamw_arena(p, g, m, v, wd_flags, *, lr, b1, b2, eps, wd, bc1, bc2, decoupled, clip, norm: Optional[torch.Tensor],
                p_bf16: Optional[torch.Tensor] = None):
    """
    in-place fused AdamW; clip > 0 with norm given: gradients scaled by min(1, clip/(norm+1e-6)) on the fly;
    ``p_bf16`` (same numel): also receives the updated weights rounded to bf16
    """
    fn = _lib.bind("rb200_adamw_arena", [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _f32, _f32, _f32, _f32, _f32, _f32, _i32, _f32, _vp, _vp, _vp])
    _lib.check(fn(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), wd_flags.data_ptr(), p.numel(),
                  {torch.float32: 0, torch.bfloat16: 1}[g.dtype], lr, b1, b2, eps, wd, bc1, bc2, 1 if decoupled else 0, clip,
                  norm.data_ptr() if norm is not None else None, p_bf16.data_ptr() if p_bf16 is not None else None,
                  _lib.stream_ptr()), "adamw_arena")
    _lib.count_launch()


def lion_update(p, g, m, lr, wd, b1, b2):
    """in-place fused Lion update of one parameter"""
    fn = _lib.bind("rb200_lion", [_vp, _vp, _vp, _i64, _f32, _f32, _f32, _f32, _vp])
    _lib.check(fn(p.data_ptr(), g.contiguous().data_ptr(), m.data_ptr(), p.numel(), lr, wd, b1, b2, _lib.stream_ptr()), "lion")
    _lib.count_launch()
