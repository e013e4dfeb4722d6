"""
Process-wide request for statically traceable model code: fixed shapes (bounded buffers, ``Dim.capacity``), fixed trip counts
with per-element gating instead of data-dependent control flow, device-side randomness, no host reads of device values.
Code written that way can be captured into a CUDA graph (``torch_cuda_graph``). Random number consumption may differ from the
default mode (bounded loops draw for gated-off iterations too).

``static_traceable_generation`` counts the off -> on transitions; the CUDA-graph train step switches the flag on once per step, so
within that regime the number identifies the step and can scope per-step caches.  Reference: returnn/frontend/static_traceable.py.
"""

from __future__ import annotations
import contextlib

__all__ = ["is_static_traceable", "set_static_traceable", "set_static_traceable_ctx", "static_traceable_generation"]

_flag = False
_generation = 0


def is_static_traceable() -> bool:
    """whether statically traceable code is requested"""
    return _flag


def set_static_traceable(flag: bool):
    """switch the request on or off"""
    global _flag, _generation
    if flag and not _flag:
        _generation += 1
    _flag = bool(flag)


def static_traceable_generation() -> int:
    """number of activations so far"""
    return _generation


@contextlib.contextmanager
def set_static_traceable_ctx(flag: bool = True):
    """the request for the duration of the block"""
    old = _flag
    try:
        set_static_traceable(flag)
        yield
    finally:
        set_static_traceable(old)
