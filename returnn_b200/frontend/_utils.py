"""
Internal helpers of the RF implementation: raw<->Tensor wrapping, dtype mapping, dim merging for broadcasting.

There is a single execution backend (torch), so RF functions call torch directly; numpy raw tensors (dataset side)
are handled by :mod:`returnn_b200.frontend._numpy_backend` for the small op set needed there.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union
import numpy
import torch
from ..tensor import Tensor, Dim, batch_dim

RawTensorTypes = Union[int, float, complex, bool, numpy.number, numpy.ndarray, str]

_TORCH_DTYPES: Dict[str, torch.dtype] = {
    "float16": torch.float16,
    "bfloat16": torch.bfloat16,
    "float32": torch.float32,
    "float64": torch.float64,
    "int8": torch.int8,
    "int16": torch.int16,
    "int32": torch.int32,
    "int64": torch.int64,
    "uint8": torch.uint8,
    "bool": torch.bool,
    "complex64": torch.complex64,
    "complex128": torch.complex128,
}
_TORCH_DTYPE_NAMES = {v: k for k, v in _TORCH_DTYPES.items()}


def torch_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    """dtype string -> torch.dtype"""
    if isinstance(dtype, torch.dtype):
        return dtype
    return _TORCH_DTYPES[dtype]


def dtype_name(dtype: torch.dtype) -> str:
    """torch.dtype -> dtype string"""
    return _TORCH_DTYPE_NAMES[dtype]


def wrap(raw: torch.Tensor, dims: Sequence[Dim], *, name: str = "tensor", sparse_dim: Optional[Dim] = None,
         feature_dim=None, like: Optional[Tensor] = None) -> Tensor:
    """
    Fast Tensor construction without the shape checks of the public constructor.

    :param like: take sparse_dim / feature_dim from here when they still apply
    """
    t = Tensor.__new__(Tensor)
    t.name = name
    t._dims = tuple(dims)
    t.dtype = _TORCH_DTYPE_NAMES[raw.dtype]
    t.version = 2
    t.control_flow_ctx = None
    t.available_for_inference = True
    t._extra = None
    t._raw_tensor = raw
    from ..utils.basic import NotSpecified

    if like is not None:
        sd = like.sparse_dim if sparse_dim is None else sparse_dim
        t.sparse_dim = sd if (sd is not None and not raw.dtype.is_floating_point and raw.dtype != torch.bool) else None
        fd = like._feature_dim
        if fd is not NotSpecified and fd is not None and fd not in t._dims:
            fd = NotSpecified
        t._feature_dim = fd if feature_dim is None else feature_dim
    else:
        t.sparse_dim = sparse_dim
        t._feature_dim = NotSpecified if feature_dim is None else feature_dim
    return t


def merge_dims_for_broadcast(a: Tensor, b: Tensor) -> Tuple[Dim, ...]:
    """
    Out dims of a binary op: the operand with more dims leads; dims only in the other one are appended
    in the order they appear there... but if one operand's dims are a superset of the other's, its order is kept.
    """
    ad, bd = a._dims, b._dims
    if ad == bd:
        return ad
    if not bd:
        return ad
    if not ad:
        return bd
    if len(bd) > len(ad) and all(d in bd for d in ad):
        return bd
    if all(d in ad for d in bd):
        return ad
    if all(d in bd for d in ad):
        return bd
    out = list(ad)
    for d in bd:
        if d not in out:
            out.append(d)
    return tuple(out)


def convert_to_tensor(value, *, dims: Optional[Sequence[Dim]] = None, dtype: Optional[str] = None, sparse_dim: Optional[Dim] = None,
                      feature_dim: Optional[Dim] = None, device: Optional[str] = None, name: Optional[str] = None,
                      like: Optional[Tensor] = None) -> Tensor:
    """
    python scalar / numpy / torch / Tensor -> Tensor. Without ``dims``, an array or raw tensor gets new static dims, one per axis,
    sized by its shape (reference: returnn/frontend/array_.py:120-140); a scalar has no dims.
    """
    if isinstance(value, Tensor):
        return value
    if dims is None:
        shape = tuple(value.shape) if isinstance(value, (torch.Tensor, numpy.ndarray)) else ()
        dims = [Dim(int(n), name="%s_dim%i" % (name or "const", i)) for i, n in enumerate(shape)]
    if isinstance(value, Dim):
        return value.get_size_tensor() if value.is_dynamic() else convert_to_tensor(value.dimension, dtype=dtype or "int32", device=device)
    if like is not None:
        if device is None:
            device = like.device
        if dtype is None and isinstance(value, (int, float, bool)):
            # python scalars adapt to the dtype of the other operand (float scalar + int tensor -> float32)
            if isinstance(value, bool):
                dtype = "bool"
            elif isinstance(value, int):
                dtype = like.dtype if like.dtype != "bool" else "int32"
            else:
                dtype = like.dtype if like.is_float() else get_default_float_dtype()
    if isinstance(value, torch.Tensor):
        raw = value
        if dtype is not None and _TORCH_DTYPE_NAMES[raw.dtype] != dtype:
            raw = raw.to(torch_dtype(dtype))
        if device is not None and str(raw.device) != str(device):
            from ..tensor.utils import host_to_device

            raw = host_to_device(raw, device)
    else:
        if dtype is None:
            if isinstance(value, bool):
                dtype = "bool"
            elif isinstance(value, int):
                dtype = get_default_int_dtype()
            elif isinstance(value, float):
                dtype = get_default_float_dtype()
            elif isinstance(value, (numpy.ndarray, numpy.number)):
                dtype = str(value.dtype)
            else:
                raise TypeError("convert_to_tensor: cannot handle %r" % type(value))
        if isinstance(value, (bool, int, float)) and device is not None and str(device).startswith("cuda"):
            # a fill kernel instead of a host-to-device copy of one element (which would synchronise the stream)
            raw = torch.full((), value, dtype=torch_dtype(dtype), device=device)
        else:
            raw = torch.as_tensor(value, dtype=torch_dtype(dtype), device=device)
    assert raw.ndim == len(dims), "convert_to_tensor: value ndim %i but dims %r" % (raw.ndim, dims)
    return wrap(raw, dims, name=name or "const", sparse_dim=sparse_dim, feature_dim=feature_dim)


_default_float_dtype = "float32"
_default_int_dtype = "int32"
_default_array_index_dtype = "int32"


def get_default_float_dtype() -> str:
    """float32 unless overridden by config default_float_dtype"""
    return _default_float_dtype


def set_default_float_dtype(dtype: str):
    """set default float dtype"""
    global _default_float_dtype
    _default_float_dtype = dtype


def get_default_int_dtype() -> str:
    """int32"""
    return _default_int_dtype


def get_default_array_index_dtype() -> str:
    """int32"""
    return _default_array_index_dtype


def axis_of(x: Tensor, dim: Dim) -> int:
    """index of dim in x (unique)"""
    dims = x._dims
    idx = -1
    for i, d in enumerate(dims):
        if d is dim or d == dim:
            if idx >= 0:
                raise ValueError("%r: dim %r is not unique" % (x, dim))
            idx = i
    if idx < 0:
        raise ValueError("%r: dim %r not found" % (x, dim))
    return idx


def dim_value(d: Dim) -> int:
    """runtime size of d"""
    return d.get_dim_value()


def shape_of(dims: Sequence[Dim]) -> List[int]:
    """runtime shape"""
    return [d.get_dim_value() for d in dims]
