"""
CTC loss with fused log-softmax (``csrc/ctc.cu``): one CTA per sequence runs the whole alpha and beta recursion in
shared memory and writes the gradient w.r.t. the logits (softmax - posterior) directly.
"""

from __future__ import annotations
import torch
from . import _lib


def available() -> bool:
    """library present with the CTC entry point"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_ctc_loss")


def ctc_loss(logits, targets, in_lens, tgt_lens, *, blank_index: int, logits_normalized: bool = False):
    """placeholder until the kernel binding is filled in"""
    raise NotImplementedError


def supports(logits, targets) -> bool:
    """shapes handled by the kernel"""
    return False
