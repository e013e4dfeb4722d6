"""
Gradient utilities.  Parity: returnn/frontend/gradient.py (set_requires_gradient, gradient, stop_gradient,
scaled_gradient, scaled_gradient_ext, gradient_checkpoint_scope).
"""

from __future__ import annotations
from typing import Optional, Union
import torch
from ..tensor import Tensor
from ._utils import wrap

__all__ = ["set_requires_gradient", "gradient", "stop_gradient", "stop_gradient_scope", "scaled_gradient",
           "scaled_gradient_ext", "gradient_checkpoint_scope"]


def set_requires_gradient(source: Tensor):
    """mark so that rf.gradient w.r.t. it works"""
    source._raw_tensor.requires_grad_(True)


def gradient(y: Tensor, x: Tensor) -> Tensor:
    """d sum(y) / dx"""
    (g,) = torch.autograd.grad(y._raw_tensor.sum(), x._raw_tensor, retain_graph=True)
    return wrap(g, x._dims, like=x)


def stop_gradient(source: Tensor) -> Tensor:
    """detach"""
    return wrap(source._raw_tensor.detach(), source._dims, like=source)


def stop_gradient_scope():
    """no_grad context"""
    return torch.no_grad()


class _ScaledGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, scale_shift_by_sum_over_axis):
        ctx.scale = scale
        ctx.shift = shift
        ctx.axis = scale_shift_by_sum_over_axis
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        out = g
        if ctx.scale is not None and not (isinstance(ctx.scale, (int, float)) and ctx.scale == 1):
            out = out * ctx.scale
        if ctx.shift is not None:
            shift = ctx.shift
            if ctx.axis is not None:
                shift = shift * g.sum(dim=ctx.axis, keepdim=True)
            out = out + shift
        return out, None, None, None


def scaled_gradient(source: Tensor, scale: Union[float, Tensor]) -> Tensor:
    """identity in forward; gradient multiplied by scale (-1: gradient reversal)"""
    s = scale._raw_tensor if isinstance(scale, Tensor) else scale
    return wrap(_ScaledGrad.apply(source._raw_tensor, s, None, None), source._dims, like=source)


def scaled_gradient_ext(source: Tensor, *, scale: Union[float, Tensor] = 1.0, shift: Optional[Union[float, Tensor]] = None,
                        scale_shift_by_sum_over_axis=None) -> Tensor:
    """gradient * scale + shift (* sum of gradient over axis)"""
    from ._utils import axis_of

    s = scale.copy_compatible_to_dims_raw(source._dims) if isinstance(scale, Tensor) and scale._dims else (
        scale._raw_tensor if isinstance(scale, Tensor) else scale)
    sh = shift.copy_compatible_to_dims_raw(source._dims) if isinstance(shift, Tensor) and shift._dims else (
        shift._raw_tensor if isinstance(shift, Tensor) else shift)
    ax = axis_of(source, scale_shift_by_sum_over_axis) if scale_shift_by_sum_over_axis is not None else None
    return wrap(_ScaledGrad.apply(source._raw_tensor, s, sh, ax), source._dims, like=source)


def gradient_checkpoint_scope():
    """
    Tensors computed inside the scope are not kept for backward but recomputed.
    See :class:`returnn_b200.torch.util.gradient_checkpoint.gradient_checkpoint_scope`.
    """
    from ..torch.util.gradient_checkpoint import gradient_checkpoint_scope as scope

    return scope()
