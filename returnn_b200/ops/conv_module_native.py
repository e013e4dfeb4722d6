"""
Binding of the fused conv-module kernels (``csrc/conv_module.cu``).
"""

from __future__ import annotations
import torch
from . import _lib


def available(x) -> bool:
    """library present with the entry points"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_glu_dwconv_fwd") and x.is_cuda and x.dtype == torch.bfloat16


def supports(channels: int, kernel: int) -> bool:
    """shapes handled"""
    return False


def glu_dwconv_bn_silu(x, filt, bias, bn, pack, *, training):
    """fused"""
    raise NotImplementedError
