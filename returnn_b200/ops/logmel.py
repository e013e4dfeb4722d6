"""
Fused log-mel frontend (``csrc/logmel.cu``): framing, Hann window, 512-point DFT as a tensor-core GEMM, power,
mel projection and log in one kernel.
"""

from __future__ import annotations
from . import _lib


def available() -> bool:
    """library present with the entry point"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_logmel")


def log_mel(audio, *, sampling_rate, window, step, n_fft, n_mel, f_min, f_max, log_base):
    """placeholder until the kernel binding is filled in"""
    raise NotImplementedError
