"""
Parameter initializers.  Parity: returnn/frontend/init.py (Normal, VarianceScaling, Glorot, He/HeNormal/HeUniform).
"""

from __future__ import annotations
from typing import Optional, Sequence, Union
import math
from ..tensor import Tensor, Dim
from . import rand as _rand

__all__ = ["ParamInit", "ParamInitType", "Normal", "VarianceScaling", "Glorot", "He", "HeNormal", "HeUniform", "Uniform", "Constant"]


class ParamInit:
    """API: ``__call__(dims, dtype, sparse_dim=None, device=None) -> Tensor | number``"""

    def __call__(self, dims: Sequence[Dim], dtype: str, sparse_dim: Optional[Dim] = None, device: Optional[str] = None,
                 out: Optional[Tensor] = None):
        raise NotImplementedError


ParamInitType = Union[Tensor, int, float, ParamInit]


class Constant(ParamInit):
    """constant value"""

    def __init__(self, value):
        self.value = value

    def __call__(self, dims, dtype, sparse_dim=None, device=None, out=None):
        return self.value


class Normal(ParamInit):
    """(truncated) normal"""

    def __init__(self, stddev: float, *, truncated: bool = True, dtype: Optional[str] = None):
        self.stddev = stddev
        self.truncated = truncated
        self.dtype = dtype
        if self.stddev <= 0.0:
            raise ValueError("Argument `stddev` must be a positive float. Received: %s" % self.stddev)

    def __call__(self, dims, dtype, sparse_dim=None, device=None, out=None):
        dtype = self.dtype or dtype
        return _rand.random(distribution="truncated_normal" if self.truncated else "normal", static=True, dims=dims,
                            mean=0.0, stddev=self.stddev, dtype=dtype, device=device)


class Uniform(ParamInit):
    """uniform in [minval, maxval)"""

    def __init__(self, minval: float = -1.0, maxval: float = 1.0):
        self.minval, self.maxval = minval, maxval

    def __call__(self, dims, dtype, sparse_dim=None, device=None, out=None):
        return _rand.random(distribution="uniform", static=True, dims=dims, minval=self.minval, maxval=self.maxval, dtype=dtype, device=device)


class VarianceScaling(ParamInit):
    """
    stddev = sqrt(scale / n) with n = fan_in / fan_out / average. For a weight ``[in, out]`` fan_in is the first dim,
    fan_out the last; for conv filters ``[out, in, *spatial]`` the receptive field size multiplies both.
    """

    scale = 1.0
    mode = "fan_in"
    distribution = "truncated_normal"
    dtype: Optional[str] = None

    def __init__(self, scale: float = None, mode: str = None, distribution: str = None, dtype: str = None):
        if scale is not None:
            self.scale = scale
        if mode is not None:
            self.mode = mode
        if distribution is not None:
            self.distribution = distribution
        if dtype is not None:
            self.dtype = dtype
        if self.scale <= 0.0:
            raise ValueError("Argument `scale` must be a positive float. Received: %s" % self.scale)
        if self.mode not in {"fan_in", "fan_out", "fan_avg"}:
            raise ValueError("Argument `mode` should be one of ('fan_in', 'fan_out', 'fan_avg'). Received: %s" % self.mode)
        if self.distribution not in {"uniform", "truncated_normal", "normal", "untruncated_normal"}:
            raise ValueError("invalid distribution %r" % self.distribution)

    def __call__(self, dims, dtype, sparse_dim=None, device=None, out=None):
        dtype = self.dtype or dtype
        fan_in, fan_out = _compute_fans(dims)
        scale = self.scale
        if self.mode == "fan_in":
            scale /= max(1.0, fan_in)
        elif self.mode == "fan_out":
            scale /= max(1.0, fan_out)
        else:
            scale /= max(1.0, (fan_in + fan_out) / 2.0)
        if self.distribution in ("truncated_normal",):
            # constant from scipy.stats.truncnorm.std(a=-2, b=2, loc=0., scale=1.)
            stddev = math.sqrt(scale) / 0.87962566103423978
            return _rand.random(distribution="truncated_normal", static=True, dims=dims, mean=0.0, stddev=stddev, dtype=dtype, device=device)
        if self.distribution in ("normal", "untruncated_normal"):
            return _rand.random(distribution="normal", static=True, dims=dims, mean=0.0, stddev=math.sqrt(scale), dtype=dtype, device=device)
        limit = math.sqrt(3.0 * scale)
        return _rand.random(distribution="uniform", static=True, dims=dims, minval=-limit, maxval=limit, dtype=dtype, device=device)


class Glorot(VarianceScaling):
    """Xavier: fan_avg, uniform"""

    scale = 1.0
    mode = "fan_avg"
    distribution = "uniform"


class He(VarianceScaling):
    """Kaiming: scale 2, fan_in, normal"""

    scale = 2.0
    mode = "fan_in"
    distribution = "normal"


HeNormal = He


class HeUniform(He):
    """Kaiming uniform"""

    distribution = "uniform"


def _compute_fans(dims: Sequence[Dim]):
    dims = [d.dimension for d in dims]
    if len(dims) < 1:
        return 1.0, 1.0
    if len(dims) == 1:
        return float(dims[0]), float(dims[0])
    if len(dims) == 2:
        return float(dims[0]), float(dims[1])
    # conv filter [out, in, *spatial]
    receptive = 1
    for d in dims[2:]:
        receptive *= d
    return float(dims[1] * receptive), float(dims[0] * receptive)
