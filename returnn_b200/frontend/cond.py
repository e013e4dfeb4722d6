"""
``rf.cond``: eager execution picks the branch on the host.  Parity: returnn/frontend/cond.py.
"""

from __future__ import annotations
from typing import Callable, TypeVar, Union
from ..tensor import Tensor

__all__ = ["cond"]
T = TypeVar("T")


def cond(pred: Union[bool, Tensor], true_fn: Callable[[], T], false_fn: Callable[[], T]) -> T:
    """``true_fn() if pred else false_fn()``; a Tensor pred must be a scalar"""
    if isinstance(pred, Tensor):
        assert not pred.dims, "rf.cond: pred must be a scalar, got %r" % pred
        pred = bool(pred.raw_tensor)
    return true_fn() if pred else false_fn()
