"""
Piecewise linear schedules.  Parity: returnn/frontend/piecewise_linear.py, stepwise_scheduler.py.
"""

from __future__ import annotations
from typing import Dict, Optional, Union
import numpy
import torch
from ..tensor import Tensor, Dim
from .module import Module
from ._utils import wrap

__all__ = ["PiecewiseLinear", "PiecewiseLinearStepwiseScheduler"]


class PiecewiseLinear(Module):
    """y(x) interpolated linearly between the given points, constant outside"""

    def __init__(self, points: Dict[Union[int, float], Union[float, Tensor]], *, kind: str = "linear",
                 ignore_first_steps: bool = False):
        super().__init__()
        if not points:
            raise ValueError("PiecewiseLinear: points must not be empty")
        self._points_sorted = sorted(points.items())
        self.kind = kind
        self.xs = numpy.array([float(x) for x, _ in self._points_sorted])
        self.ys = numpy.array([float(y) for _, y in self._points_sorted])

    def __call__(self, x: Union[Tensor, int, float]) -> Union[Tensor, float]:
        if isinstance(x, Tensor):
            raw = x.raw_tensor.to(torch.float32)
            xs = torch.tensor(self.xs, dtype=torch.float32, device=raw.device)
            ys = torch.tensor(self.ys, dtype=torch.float32, device=raw.device)
            idx = torch.searchsorted(xs, raw.contiguous(), right=True).clamp(1, len(self.xs) - 1) if len(self.xs) > 1 else None
            if idx is None:
                return wrap(torch.full_like(raw, float(self.ys[0])), x.dims)
            x0, x1, y0, y1 = xs[idx - 1], xs[idx], ys[idx - 1], ys[idx]
            t = ((raw - x0) / (x1 - x0)).clamp(0, 1)
            if self.kind == "flat":
                t = torch.floor(t)
            return wrap(y0 + t * (y1 - y0), x.dims)
        if self.kind == "flat":
            i = int(numpy.searchsorted(self.xs, float(x), side="right")) - 1
            return float(self.ys[max(i, 0)])
        return float(numpy.interp(float(x), self.xs, self.ys))


class PiecewiseLinearStepwiseScheduler(PiecewiseLinear):
    """PiecewiseLinear evaluated at the current global train step"""

    def __call__(self) -> Union[Tensor, float]:
        from .run_ctx import get_run_ctx

        return super().__call__(get_run_ctx().step)
