"""
``State``: nested container for recurrent state (attribute and item access; tree-mappable).
Parity: returnn/frontend/state.py:14.
"""

from __future__ import annotations
from typing import Any, Dict

__all__ = ["State"]


class State(dict):
    """
    dict with attribute access. ``State(h=..., c=...)`` or ``State({0: ..., 1: ...})`` or ``State(x)`` for one positional.
    """

    def __init__(self, *args, **kwargs):
        if kwargs:
            assert not args
            super().__init__(**kwargs)
        elif args:
            assert len(args) == 1
            if isinstance(args[0], dict):
                super().__init__(args[0])
            else:
                super().__init__()
                self["_"] = args[0]
        else:
            super().__init__()

    def __repr__(self):
        return "%s(%s)" % (self.__class__.__name__, ", ".join("%s=%r" % (k, v) for k, v in self.items()))

    def __getattr__(self, item):
        if item in self:
            return self[item]
        raise AttributeError("%s has no attribute %r" % (self.__class__.__name__, item))

    def __setattr__(self, key, value):
        self[key] = value

    def flatten_tensors(self):
        """all leaves"""
        from .nested import tree_flatten

        return tree_flatten(self)

    def deep_tensors(self):
        """alias"""
        return self.flatten_tensors()
