"""
Softmax cross entropy with label smoothing over a large vocabulary, one online-softmax pass per row.
"""

from __future__ import annotations
import ctypes
import torch
from . import _lib

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def available() -> bool:
    """native library has the kernel"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_softmax_ce_fwd")


class _CeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, smoothing):
        logits = logits.contiguous()
        rows, v = logits.shape
        tgt = targets.to(torch.int32).contiguous()
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        fn = _lib.bind("rb200_softmax_ce_fwd", [_vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _vp])
        _lib.check(fn(logits.data_ptr(), tgt.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows, v, smoothing,
                      1 if logits.dtype == torch.bfloat16 else 0, _lib.stream_ptr()), "softmax_ce_fwd")
        _lib.count_launch()
        ctx.save_for_backward(logits, tgt, lse)
        ctx.smoothing = smoothing
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, tgt, lse = ctx.saved_tensors
        rows, v = logits.shape
        dlogits = torch.empty_like(logits)
        dl = dloss.to(torch.float32).contiguous()
        fn = _lib.bind("rb200_softmax_ce_bwd", [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _vp])
        _lib.check(fn(logits.data_ptr(), tgt.data_ptr(), lse.data_ptr(), dl.data_ptr(), dlogits.data_ptr(), rows, v,
                      ctx.smoothing, 1 if logits.dtype == torch.bfloat16 else 0, _lib.stream_ptr()), "softmax_ce_bwd")
        _lib.count_launch()
        return dlogits, None, None


def softmax_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0) -> torch.Tensor:
    """
    :param logits: [rows, V] bf16 or fp32
    :param targets: [rows] int
    :param label_smoothing: target distribution (1-s) one-hot + s/(V-1) elsewhere
    :return: [rows] fp32 loss
    """
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and _lib.use_native(logits) and available():
        return _CeFn.apply(logits, targets, float(label_smoothing))
    return softmax_cross_entropy_reference(logits, targets, label_smoothing)


def softmax_cross_entropy_reference(logits, targets, label_smoothing=0.0):
    """plain torch in fp32"""
    lp = torch.log_softmax(logits.float(), dim=-1)
    nll = -lp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    if not label_smoothing:
        return nll
    v = logits.shape[-1]
    other = (-lp.sum(dim=-1) - nll) / (v - 1)
    return (1.0 - label_smoothing) * nll + label_smoothing * other
