"""
Current control-flow scope (bookkeeping only; execution is eager).  Parity: returnn/frontend/control_flow_ctx.py.
"""

from __future__ import annotations
from typing import Optional
import contextlib
from ..tensor import ControlFlowContext

_ctx: Optional[ControlFlowContext] = None


def get_current_control_flow_ctx() -> Optional[ControlFlowContext]:
    """innermost scope or None"""
    return _ctx


@contextlib.contextmanager
def control_flow_ctx(ctx: Optional[ControlFlowContext] = None):
    """enter a scope"""
    global _ctx
    prev = _ctx
    _ctx = ctx
    try:
        yield ctx
    finally:
        _ctx = prev
