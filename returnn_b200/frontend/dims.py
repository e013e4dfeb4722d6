"""
Dim-related functions: ranges, size tensors, replacing dims, dim matching helpers.

Parity: returnn/frontend/dims.py.
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap, torch_dtype, axis_of

__all__ = ["range_over_dim", "range_over_dim_strided", "range_over_merged_dims", "linspace_over_dim", "replace_dim",
           "replace_dim_v2", "set_sparse_dim", "dim_match_priority_when_needed", "num_elements_of_shape",
           "masked_fraction_of_shape", "last_frame_position_of_dim", "use_mask_default", "length"]


def range_over_dim(dim: Dim, *, dtype: Optional[str] = None, device: Optional[str] = None) -> Tensor:
    """[0, 1, ..., dim-1] with sparse_dim=dim"""
    if device is None:
        from .device import get_default_device

        device = get_default_device()
    raw = torch.arange(dim.get_dim_value(), dtype=torch_dtype(dtype or "int32"), device=device)
    return wrap(raw, [dim], sparse_dim=dim if not (dtype or "int32").startswith("float") else None)


def range_over_dim_strided(dim: Dim, *, stride: int, out_dim: Optional[Dim] = None, dtype=None, device=None) -> Tuple[Tensor, Dim]:
    """[0, stride, 2*stride, ...] < dim"""
    if out_dim is None:
        out_dim = dim.ceildiv_right(stride)
    r = range_over_dim(out_dim, dtype=dtype, device=device)
    return wrap(r._raw_tensor * stride, [out_dim], sparse_dim=dim), out_dim


def range_over_merged_dims(dims: Sequence[Dim], *, dtype=None, device=None) -> Tensor:
    """flat index over several dims, shaped by those dims"""
    shape = [d.get_dim_value() for d in dims]
    n = 1
    for s in shape:
        n *= s
    raw = torch.arange(n, dtype=torch_dtype(dtype or "int32"), device=device).reshape(shape)
    return wrap(raw, list(dims))


def linspace_over_dim(dim: Dim, start=0.0, end=1.0, *, dtype=None, device=None) -> Tensor:
    """linspace with dim points"""
    raw = torch.linspace(float(start), float(end), dim.get_dim_value(), dtype=torch_dtype(dtype or "float32"), device=device)
    return wrap(raw, [dim])


def replace_dim(source: Tensor, *, in_dim: Dim, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """rename an axis (sizes must agree)"""
    if out_dim is None:
        out_dim = in_dim.copy(same_as_self=False, description="new-dim")
    ax = axis_of(source, in_dim)
    dims = list(source._dims)
    dims[ax] = out_dim
    res = wrap(source._raw_tensor, dims, like=source)
    if source.feature_dim == in_dim:
        res._feature_dim = out_dim
    if out_dim.is_dynamic() and out_dim.dyn_size_ext is None and in_dim.dyn_size_ext is not None:
        out_dim.dyn_size_ext = in_dim.dyn_size_ext
    return res, out_dim


def replace_dim_v2(source: Tensor, *, in_dim: Dim, out_dim: Dim, allow_expand: bool = True, allow_shrink: bool = True) -> Tensor:
    """rename an axis, padding or cutting when the new dim is longer or shorter"""
    ax = axis_of(source, in_dim)
    n_in = source._raw_tensor.shape[ax]
    n_out = out_dim.get_dim_value()
    raw = source._raw_tensor
    if n_out > n_in:
        assert allow_expand
        raw = torch.nn.functional.pad(raw, [0, 0] * (raw.ndim - ax - 1) + [0, n_out - n_in])
    elif n_out < n_in:
        assert allow_shrink
        raw = raw.narrow(ax, 0, n_out)
    dims = list(source._dims)
    dims[ax] = out_dim
    return wrap(raw, dims, like=source)


def set_sparse_dim(source: Tensor, sparse_dim: Dim) -> Tensor:
    """copy with other sparse dim"""
    res = source.copy()
    res.sparse_dim = sparse_dim
    return res


def dim_match_priority_when_needed(dim: Dim, *other_dims: Dim) -> Dim:
    """dims are matched by identity here, so no priority is needed"""
    return dim


def num_elements_of_shape(dims, *, use_mask: bool = True, device=None):
    """see rf.array_.num_elements_of_shape"""
    from .array_ import num_elements_of_shape as f

    return f(dims, use_mask=use_mask, device=device)


def masked_fraction_of_shape(dims: Union[Dim, Sequence[Dim]], *, inverse: bool = False) -> float:
    """valid / total elements (or total / valid)"""
    if isinstance(dims, Dim):
        dims = [dims]
    n_valid = num_elements_of_shape(dims, use_mask=True)
    n_total = 1
    for d in dims:
        n_total *= d.get_dim_value()
    return (n_total / max(n_valid, 1)) if inverse else (n_valid / max(n_total, 1))


def last_frame_position_of_dim(dim: Dim, *, device=None, allow_scalar_on_cpu: bool = True) -> Union[int, Tensor]:
    """size - 1, clipped at 0"""
    if dim.is_static():
        return max(dim.dimension - 1, 0)
    sizes = dim.get_size_tensor(device=device)
    return wrap((sizes._raw_tensor - 1).clamp_min(0), sizes._dims, sparse_dim=dim)


def use_mask_default(*, default: Optional[bool] = None, default_false_for_behavior_version_up_to: Optional[int] = None, func_name=None) -> Optional[bool]:
    """global default for use_mask: config ``rf_use_mask``"""
    from ..config import get_global_config

    cfg = get_global_config(raise_exception=False)
    if cfg and cfg.has("rf_use_mask"):
        return cfg.bool("rf_use_mask", True)
    if default_false_for_behavior_version_up_to is not None:
        from ..utils.basic import BehaviorVersion

        if BehaviorVersion.get() <= default_false_for_behavior_version_up_to:
            return False
    return default


def length(dim: Dim, *, dtype=None, device=None):
    """sizes of dim as Tensor or int"""
    if dim.is_static():
        return dim.dimension
    return dim.get_size_tensor(device=device)
