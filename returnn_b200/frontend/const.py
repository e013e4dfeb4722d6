"""
Constant tensors.

Parity: returnn/frontend/const.py.
"""

from __future__ import annotations
from typing import Optional, Sequence, Union
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap, torch_dtype, get_default_float_dtype, shape_of

__all__ = ["full", "constant", "fill", "zeros", "ones", "zeros_like", "ones_like", "full_like"]


def full(*, dims: Sequence[Dim], fill_value, dtype: Optional[str] = None, device: Optional[str] = None,
         sparse_dim: Optional[Dim] = None, feature_dim: Optional[Dim] = None) -> Tensor:
    """tensor of dims filled with fill_value"""
    if isinstance(fill_value, Tensor):
        fill_value = fill_value._raw_tensor.item()
    if dtype is None:
        if isinstance(fill_value, bool):
            dtype = "bool"
        elif isinstance(fill_value, int):
            dtype = "int32"
        else:
            dtype = get_default_float_dtype()
    if device is None:
        from .device import get_default_device

        device = get_default_device()
    raw = torch.full(shape_of(dims), fill_value, dtype=torch_dtype(dtype), device=device)
    return wrap(raw, dims, sparse_dim=sparse_dim, feature_dim=feature_dim)


constant = full
fill = full


def zeros(dims: Sequence[Dim], *, dtype=None, device=None, sparse_dim=None, feature_dim=None) -> Tensor:
    """zeros"""
    return full(dims=dims, fill_value=0 if (dtype or "").startswith("int") else (False if dtype == "bool" else 0.0),
                dtype=dtype or get_default_float_dtype(), device=device, sparse_dim=sparse_dim, feature_dim=feature_dim)


def ones(dims: Sequence[Dim], *, dtype=None, device=None, sparse_dim=None, feature_dim=None) -> Tensor:
    """ones"""
    return full(dims=dims, fill_value=1 if (dtype or "").startswith("int") else (True if dtype == "bool" else 1.0),
                dtype=dtype or get_default_float_dtype(), device=device, sparse_dim=sparse_dim, feature_dim=feature_dim)


def zeros_like(other: Tensor) -> Tensor:
    """zeros with other's meta"""
    return wrap(torch.zeros_like(other._raw_tensor), other._dims, like=other)


def ones_like(other: Tensor) -> Tensor:
    """ones with other's meta"""
    return wrap(torch.ones_like(other._raw_tensor), other._dims, like=other)


def full_like(other: Tensor, fill_value) -> Tensor:
    """filled with other's meta"""
    return wrap(torch.full_like(other._raw_tensor, fill_value), other._dims, like=other)
