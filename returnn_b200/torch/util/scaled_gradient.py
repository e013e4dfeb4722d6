"""
Identity in the forward pass, scaled (or clipped/shifted) gradient in the backward pass.

Parity: returnn/torch/util/scaled_gradient.py (scaled_gradient :44, scaled_gradient_ext :92).
"""

from __future__ import annotations
from typing import Optional, Union
import torch


class _Scale(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.scale, None


def scaled_gradient(x: torch.Tensor, scale: float) -> torch.Tensor:
    """:return: x, with d/dx multiplied by ``scale`` (``scale = -1``: gradient reversal)"""
    return _Scale.apply(x, scale)


class _ScaleExt(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, lower, upper):
        ctx.args = (scale, shift, lower, upper)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        scale, shift, lower, upper = ctx.args
        g = g * scale
        if shift is not None:
            g = g + shift
        if lower is not None or upper is not None:
            g = torch.clamp(g, min=lower, max=upper)
        return g, None, None, None, None


def scaled_gradient_ext(x: torch.Tensor, *, scale: Union[float, torch.Tensor] = 1.0, shift: Optional[Union[float, torch.Tensor]] = None,
                        scale_shift_by_sum_over_axis: Optional[int] = None) -> torch.Tensor:
    """
    :param scale: factor on the gradient
    :param shift: added to the scaled gradient
    :param scale_shift_by_sum_over_axis: if given, scale and shift are first multiplied by the sum of the gradient over that axis
    :return: x with the modified gradient
    """
    if scale_shift_by_sum_over_axis is None:
        return _ScaleExt.apply(x, scale, shift, None, None)

    class _BySum(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x_):
            return x_.view_as(x_)

        @staticmethod
        def backward(ctx, g):
            m = g.sum(dim=scale_shift_by_sum_over_axis, keepdim=True)
            out = g * (scale * m)
            if shift is not None:
                out = out + shift * m
            return out

    return _BySum.apply(x)
