"""Type aliases of the frontend API (reference: returnn/frontend/types.py)."""

from __future__ import annotations
from typing import Protocol, Sequence, Type, Union
import numpy
from ..tensor import Tensor, Dim, TensorDict

__all__ = ["RawTensorTypes", "ItemKeyType", "Tensor", "Dim", "get_raw_tensor_type", "GetModelFunc", "StepFunc"]

RawTensorTypes = Union[int, float, complex, numpy.number, numpy.ndarray, bool, str]
ItemKeyType = Union[RawTensorTypes, Tensor, slice, Sequence[Union[RawTensorTypes, Tensor, slice]]]


class GetModelFunc(Protocol):
    """``get_model`` of a config"""

    def __call__(self, *, epoch: int, step: int): ...


class StepFunc(Protocol):
    """``train_step`` / ``forward_step`` of a config"""

    def __call__(self, *, model, extern_data: TensorDict) -> None: ...


def get_raw_tensor_type() -> Type:
    """the raw tensor type behind :class:`Tensor`: ``torch.Tensor``"""
    import torch

    return torch.Tensor
