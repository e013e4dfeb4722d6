"""Encoder interfaces.  Parity: returnn/frontend/encoder/base.py."""

from __future__ import annotations
from typing import Tuple, Union
from ...tensor import Tensor, Dim
from ..module import Module


class IEncoder(Module):
    """x -> y with same spatial dims"""

    out_dim: Dim

    def __call__(self, source: Tensor) -> Tensor:
        raise NotImplementedError


class ISeqFramewiseEncoder(Module):
    """(x, spatial_dim) -> y, frame-wise"""

    out_dim: Dim

    def __call__(self, source: Tensor, *, spatial_dim: Dim) -> Tensor:
        raise NotImplementedError


class ISeqDownsamplingEncoder(Module):
    """(x, in_spatial_dim) -> (y, out_spatial_dim)"""

    out_dim: Dim
    downsample_factor: Union[int, float]

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim) -> Tuple[Tensor, Dim]:
        raise NotImplementedError
