"""
Asynchronous device-side assertion.

On CUDA the condition is checked by a one-thread kernel that writes a status word into pinned host memory
(:func:`returnn_b200.ops.seq_ops.device_assert`); nothing traps on the device, so the context stays usable. With
``stop=True`` the failure is raised at the next :func:`check_pending` (call it once per step): a kernel cannot raise a
Python exception at the moment it runs.

Parity: returnn/torch/util/assert_.py (assert_ :13; the reference launches a kernel that prints and traps).
"""

from __future__ import annotations
from typing import List
import torch

_warn_only: List[str] = []


def assert_(cond: torch.Tensor, message: str, *, stop: bool = True):
    """
    :param cond: bool tensor (all elements must be true)
    :param message: shown when the condition is false
    :param stop: raise (CPU: at once; CUDA: at the next :func:`check_pending`); otherwise print a warning
    """
    if type(cond) is not torch.Tensor:
        return  # traced / fake tensor: no storage to check
    if cond.device.type == "cpu":
        if not bool(cond.all()):
            if stop:
                raise AssertionError(message)
            print("[ASSERT FAILED WARNING]: %s" % message)
        return
    if cond.device.type != "cuda":
        raise NotImplementedError("assert_ on device type %r" % cond.device.type)
    if torch.cuda.is_current_stream_capturing():
        return  # the eager warm-up steps before a capture ran the check already
    from ...ops import seq_ops

    if not stop:
        _warn_only.append(message)
    seq_ops.device_assert(cond, message)


def check_pending(*, wait: bool = False):
    """
    Read the status words written so far (``wait``: synchronise the device first).

    :raises AssertionError: for a failed assertion that was registered with ``stop=True``
    """
    from ...ops import seq_ops

    if wait and torch.cuda.is_available():
        torch.cuda.synchronize()
    try:
        seq_ops.check_asserts()
    except AssertionError as exc:
        if any(str(exc).startswith(m) for m in _warn_only):
            print("[ASSERT FAILED WARNING]: %s" % exc)
            return
        raise
