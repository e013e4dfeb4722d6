"""
``rf.assert_``: check a condition without stalling the device. A Python bool is checked at once; a tensor condition is reduced to
a scalar and handed to the asynchronous device assert (:mod:`returnn_b200.torch.util.assert_`: a one-thread kernel writes a
status word into pinned host memory, the host raises when it next looks; no trap, the CUDA context survives).
Reference: returnn/frontend/assert_.py.
"""

from __future__ import annotations
from typing import Union
from ..tensor import Tensor

__all__ = ["assert_"]


def assert_(condition: Union[Tensor, bool], message: str, *, stop: bool = True) -> None:
    """
    :param condition: bool, or a bool tensor (all elements must hold)
    :param message: text of the error
    :param stop: raise ``AssertionError`` (True) or only print a warning (False)
    """
    if isinstance(condition, bool):
        if not condition:
            if stop:
                raise AssertionError(message)
            print("[ASSERT FAILED WARNING]: %s" % message)
        return
    if not isinstance(condition, Tensor):
        raise TypeError("assert_: condition must be a bool or a Tensor, got %r" % type(condition))
    raw = condition.raw_tensor
    if raw.ndim:
        raw = raw.all()
    from ..torch.util.assert_ import assert_ as _device_assert

    _device_assert(raw, message, stop=stop)
