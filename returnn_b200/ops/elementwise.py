"""
Fused element-wise kernels on bf16: dropout with a replayable counter-based RNG (philox keyed on a device-resident
seed and the element index, so CUDA-graph replays draw fresh masks when the seed tensor is advanced on device).
"""

from __future__ import annotations
import ctypes
import torch
from . import _lib

_vp, _i64, _f32 = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float
_seed_state = {}


def available() -> bool:
    """native library loaded"""
    return _lib.get_lib() is not None and hasattr(_lib.get_lib(), "rb200_dropout_bf16")


def _seed_tensor(device) -> torch.Tensor:
    key = str(device)
    t = _seed_state.get(key)
    if t is None:
        t = torch.zeros(2, dtype=torch.int64, device=device)
        t[0] = torch.initial_seed() % (2 ** 62)
        _seed_state[key] = t
    return t


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p):
        x = x.contiguous()
        y = torch.empty_like(x)
        seed = _seed_tensor(x.device)
        # offset advances on device: replay-safe
        off = seed[1:2].clone()
        seed[1] += x.numel()
        fn = _lib.bind("rb200_dropout_bf16", [_vp, _vp, _i64, _f32, _vp, _vp, _vp])
        _lib.check(fn(x.data_ptr(), y.data_ptr(), x.numel(), p, seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "dropout")
        _lib.count_launch()
        ctx.p = p
        ctx.save_for_backward(off)
        return y

    @staticmethod
    def backward(ctx, dy):
        (off,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(dy)
        seed = _seed_tensor(dy.device)
        fn = _lib.bind("rb200_dropout_bf16", [_vp, _vp, _i64, _f32, _vp, _vp, _vp])
        _lib.check(fn(dy.data_ptr(), dx.data_ptr(), dy.numel(), ctx.p, seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "dropout_bwd")
        _lib.count_launch()
        return dx, None


def dropout(x: torch.Tensor, p: float) -> torch.Tensor:
    """bf16 dropout, scale 1/(1-p)"""
    return _DropoutFn.apply(x, float(p))


def dropout_with_state(x: torch.Tensor, p: float, seed: torch.Tensor, offset: torch.Tensor) -> torch.Tensor:
    """
    dropout with an explicit RNG state: int64 device tensors ``seed`` (key) and ``offset`` (counter of element 0).
    Element ``i`` of the flattened input uses counter ``offset + i``, which is also what the fused GEMM epilogue and the
    native encoder kernels use, so a mask can be re-created by any of them.
    """
    x = x.contiguous()
    y = torch.empty_like(x)
    seed = seed.contiguous()
    offset = offset.contiguous()
    fn = _lib.bind("rb200_dropout_bf16", [_vp, _vp, _i64, _f32, _vp, _vp, _vp])
    _lib.check(fn(x.data_ptr(), y.data_ptr(), x.numel(), float(p), seed.data_ptr(), offset.data_ptr(), _lib.stream_ptr()), "dropout")
    _lib.count_launch()
    return y
