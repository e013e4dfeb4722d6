"""
Default dtypes.  Parity: returnn/frontend/dtype.py.
"""

from __future__ import annotations
from ._utils import (get_default_float_dtype, set_default_float_dtype, get_default_int_dtype,
                     get_default_array_index_dtype)

__all__ = ["get_default_float_dtype", "set_default_float_dtype", "set_default_float_dtype_ctx", "get_default_int_dtype",
           "get_default_array_index_dtype", "is_float_dtype", "is_int_dtype"]


def is_float_dtype(dtype: str) -> bool:
    """float16/bfloat16/float32/float64"""
    return dtype.startswith("float") or dtype == "bfloat16"


def is_int_dtype(dtype: str) -> bool:
    """signed or unsigned int"""
    return dtype.startswith("int") or dtype.startswith("uint")


import contextlib as _contextlib


@_contextlib.contextmanager
def set_default_float_dtype_ctx(dtype: str):
    """default float dtype (of new parameters, constants, random tensors) for the duration of the block"""
    assert isinstance(dtype, str)
    old = get_default_float_dtype()
    try:
        set_default_float_dtype(dtype)
        yield
    finally:
        set_default_float_dtype(old)
