"""
Label smoothing.  Parity: returnn/frontend/label_smoothing.py (label_smoothing, smooth_one_hot,
label_smoothed_log_prob_gradient :56-141).
"""

from __future__ import annotations
from typing import Optional, Sequence, Union
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap, axis_of

__all__ = ["label_smoothing", "smooth_one_hot", "label_smoothed_log_prob_gradient"]


def label_smoothing(prob: Tensor, smoothing: Union[Tensor, float], *, axis: Optional[Dim] = None) -> Tensor:
    """
    Sparse targets become a dense distribution with ``1 - smoothing`` on the label and ``smoothing / (n - 1)`` elsewhere;
    a dense distribution is mixed with the uniform one.
    """
    if not axis:
        axis = prob.feature_dim or prob.sparse_dim
    if prob.sparse_dim:
        assert prob.sparse_dim == axis
        from .array_ import sparse_to_dense

        return sparse_to_dense(prob, label_value=1.0 - smoothing, other_value=smoothing / (axis.dimension - 1))
    return prob * (1.0 - smoothing) + smoothing / axis.dimension


def smooth_one_hot(source: Tensor, *, label_prob: Union[Tensor, float]) -> Tensor:
    """one-hot with label_prob on the label and the rest spread uniformly"""
    assert source.sparse_dim
    from .array_ import sparse_to_dense

    return sparse_to_dense(source, label_value=label_prob, other_value=(1.0 - label_prob) / (source.sparse_dim.dimension - 1))


class _LsGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, log_probs, smoothing, axis, exclude):
        ctx.smoothing = smoothing
        ctx.axis = axis
        ctx.exclude = exclude
        return log_probs.view_as(log_probs)

    @staticmethod
    def backward(ctx, g):
        # Gradient as if the target were smoothed: dL/dlogp_v = (1-s) g_v + s/n * sum_u g_u
        n = g.shape[ctx.axis]
        if ctx.exclude is None:
            total = g.sum(dim=ctx.axis, keepdim=True)
            return (1.0 - ctx.smoothing) * g + (ctx.smoothing / n) * total, None, None, None
        mask = torch.ones(n, dtype=g.dtype, device=g.device)
        mask[list(ctx.exclude)] = 0.0
        shape = [1] * g.ndim
        shape[ctx.axis] = n
        mask = mask.reshape(shape)
        n_eff = int(mask.sum().item())
        total = (g * mask).sum(dim=ctx.axis, keepdim=True)
        smoothed = (1.0 - ctx.smoothing) * g + (ctx.smoothing / n_eff) * total
        return torch.where(mask > 0, smoothed, g), None, None, None


def label_smoothed_log_prob_gradient(log_prob: Tensor, smoothing: Union[Tensor, float], *, axis: Optional[Dim] = None,
                                     exclude_labels: Optional[Sequence[int]] = None) -> Tensor:
    """
    Identity in forward. In backward the incoming gradient is redistributed as label smoothing would:
    useful for losses (CTC, full-sum) where the target distribution is implicit.
    """
    if not isinstance(smoothing, Tensor) and smoothing == 0:
        return log_prob
    if not axis:
        axis = log_prob.feature_dim
    s = float(smoothing.raw_tensor) if isinstance(smoothing, Tensor) else float(smoothing)
    ax = axis_of(log_prob, axis)
    raw = _LsGrad.apply(log_prob._raw_tensor, s, ax, tuple(exclude_labels) if exclude_labels else None)
    return wrap(raw, log_prob._dims, like=log_prob)
