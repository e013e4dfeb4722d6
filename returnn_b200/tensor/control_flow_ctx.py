"""
Nesting of loop / cond scopes. Execution here is eager, so scopes only carry bookkeeping:
which loop a tensor was created in (used by ``rf.scan`` / ``rf.while_loop`` for sanity checks).

Parity: returnn/tensor/control_flow_ctx.py:1-188.
"""

from __future__ import annotations
from typing import Optional


class ControlFlowContext:
    """one loop or cond scope"""

    class Types:
        """kinds"""

        Loop = "loop"
        Cond = "cond"
        CondTrue = "cond-true"
        CondFalse = "cond-false"

    def __init__(self, *, kind: str, identifier: str = "", outer_ctx: Optional["ControlFlowContext"] = None):
        self.kind = kind
        self.identifier = identifier
        self.outer_ctx = outer_ctx
        self.loop_spatial_dim = None

    def __repr__(self):
        return "ControlFlowContext{%s}" % self.repr_inner()

    def repr_inner(self) -> str:
        """outer/.../self"""
        s = "%s:%s" % (self.kind, self.identifier)
        return (self.outer_ctx.repr_inner() + "/" + s) if self.outer_ctx else s

    @classmethod
    def abs_ctx_stack(cls, ctx: Optional["ControlFlowContext"]):
        """[outermost, ..., ctx]"""
        out = []
        while ctx:
            out.append(ctx)
            ctx = ctx.outer_ctx
        return out[::-1]

    @classmethod
    def abs_ctx_stack_with_root(cls, ctx):
        """[None, outermost, ..., ctx]"""
        return [None] + cls.abs_ctx_stack(ctx)

    @classmethod
    def is_parent_or_same(cls, parent, child) -> bool:
        """parent encloses child"""
        if parent is None or parent is child:
            return True
        while child:
            if child is parent:
                return True
            child = child.outer_ctx
        return False

    @classmethod
    def collect_parent_dims(cls, ctx):
        """loop dims of enclosing loops"""
        dims = []
        for c in cls.abs_ctx_stack(ctx):
            if c.is_loop() and c.loop_spatial_dim is not None:
                dims.append(c.loop_spatial_dim)
        return dims

    def is_loop(self) -> bool:
        """loop scope"""
        return self.kind == self.Types.Loop

    def is_cond(self) -> bool:
        """cond scope"""
        return self.kind in (self.Types.Cond, self.Types.CondTrue, self.Types.CondFalse)

    def outer_ctx_stack(self):
        """stack excluding self"""
        return self.abs_ctx_stack(self.outer_ctx)
