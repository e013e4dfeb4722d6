"""
bf16 GEMM on 5th-gen tensor cores (``csrc/gemm_tcgen05.cu``): TMA-fed shared-memory ring, ``tcgen05.mma`` issued by one
thread into a TMEM accumulator, epilogue warps read TMEM with ``tcgen05.ld`` and apply bias / activation / residual.

``linear_bf16`` is the autograd entry used by :func:`returnn_b200.ops.linear.linear`.
"""

from __future__ import annotations
from typing import Optional
import torch
from . import _lib


def available(x: torch.Tensor) -> bool:
    """library present with the GEMM entry point"""
    if not x.is_cuda:
        return False
    if not _lib.use_native(x):
        return False
    return hasattr(_lib.get_lib(), "rb200_gemm_bf16")


def linear_bf16(x, weight, bias, activation):
    """placeholder until the kernel binding below is filled in"""
    raise NotImplementedError
ENABLED = False
