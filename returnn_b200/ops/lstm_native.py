"""
Binding of the persistent LSTM kernel (``csrc/lstm.cu``).
"""

from __future__ import annotations
import torch
from . import _lib


def available(x) -> bool:
    """library present with the LSTM entry points"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_lstm_fwd") and x.is_cuda


def supports(x, w_rec) -> bool:
    """shapes handled by the persistent kernel"""
    return False


def lstm(x, lens, w_ff, w_rec, bias, h0, c0, reverse=False):
    """persistent-kernel LSTM"""
    raise NotImplementedError
