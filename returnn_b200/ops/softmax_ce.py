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
    def forward(ctx, logits, targets, smoothing, grad_only, with_argmax):
        logits = logits.contiguous()
        rows, v = logits.shape
        tgt = targets.to(torch.int32).contiguous()
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        amax = torch.empty(rows, dtype=torch.int32, device=logits.device) if with_argmax else None
        fn = _lib.bind("rb200_softmax_ce_fwd", [_vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _i32, _vp, _vp])
        _lib.check(fn(logits.data_ptr(), tgt.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows, v, smoothing,
                      1 if logits.dtype == torch.bfloat16 else 0, 1 if grad_only else 0, amax.data_ptr() if with_argmax else None,
                      _lib.stream_ptr()), "softmax_ce_fwd")
        _lib.count_launch()
        ctx.save_for_backward(logits, tgt, lse)
        ctx.smoothing = smoothing
        ctx.grad_only = grad_only
        if with_argmax:
            ctx.mark_non_differentiable(amax)
            return loss, amax
        return loss

    @staticmethod
    def backward(ctx, dloss, *_unused):
        logits, tgt, lse = ctx.saved_tensors
        rows, v = logits.shape
        dlogits = torch.empty_like(logits)
        dl = dloss.to(torch.float32).contiguous()
        fn = _lib.bind("rb200_softmax_ce_bwd", [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _i32, _i32, _vp])
        _lib.check(fn(logits.data_ptr(), tgt.data_ptr(), lse.data_ptr(), dl.data_ptr(), dlogits.data_ptr(), rows, v,
                      ctx.smoothing, 1 if logits.dtype == torch.bfloat16 else 0, 1 if ctx.grad_only else 0, _lib.stream_ptr()), "softmax_ce_bwd")
        _lib.count_launch()
        return dlogits, None, None, None, None


def softmax_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0, *, grad_only_smoothing: bool = False,
                          with_argmax: bool = False):
    """
    :param logits: [rows, V] bf16 or fp32
    :param targets: [rows] int
    :param label_smoothing: s. Default: the target distribution is (1-s) one-hot + s/(V-1) elsewhere.
    :param grad_only_smoothing: the loss stays the negative log likelihood; only its gradient is smoothed, uniformly over all V
        classes (dlogits = p - (1-s) one-hot - s/V): log-softmax, an identity whose backward redistributes the gradient
        (returnn/frontend/label_smoothing.py:86, label_smoothed_log_prob_gradient), gather of the target, in one pass
    :param with_argmax: also return the arg max over V per row (int32), e.g. for the frame error
    :return: [rows] fp32 loss (, [rows] int32 arg max)
    """
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and _lib.use_native(logits) and available():
        return _CeFn.apply(logits, targets, float(label_smoothing), bool(grad_only_smoothing), bool(with_argmax))
    loss = softmax_cross_entropy_reference(logits, targets, label_smoothing, grad_only_smoothing=grad_only_smoothing)
    if with_argmax:
        return loss, logits.argmax(dim=-1).to(torch.int32)
    return loss


class _SmoothGrad(torch.autograd.Function):
    """identity on log-probabilities [rows, V]; backward (1-s) g + s/V sum_v g"""

    @staticmethod
    def forward(ctx, lp, s):
        ctx.s = s
        return lp.view_as(lp)

    @staticmethod
    def backward(ctx, g):
        return (1.0 - ctx.s) * g + (ctx.s / g.shape[-1]) * g.sum(dim=-1, keepdim=True), None


def softmax_cross_entropy_reference(logits, targets, label_smoothing=0.0, *, grad_only_smoothing=False):
    """plain torch in fp32"""
    lp = torch.log_softmax(logits.float(), dim=-1)
    if grad_only_smoothing:
        if label_smoothing:
            lp = _SmoothGrad.apply(lp, float(label_smoothing))
        return -lp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    nll = -lp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    if not label_smoothing:
        return nll
    v = logits.shape[-1]
    other = (-lp.sum(dim=-1) - nll) / (v - 1)
    return (1.0 - label_smoothing) * nll + label_smoothing * other
