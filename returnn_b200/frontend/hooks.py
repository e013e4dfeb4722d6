"""
Hooks on module calls (pre-forward hooks that may rewrite args).  Parity: returnn/frontend/hooks.py.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Tuple
from types import MethodType
import weakref
from .module import Module

__all__ = ["setup_post_hook_on_method", "MethodWithHooks", "RemovableHandle", "setup_pre_hook_on_method"]


class RemovableHandle:
    """returned by hook registration; ``remove()`` unregisters"""

    _next_id = 0

    def __init__(self, hooks_dict: Dict[int, Callable], on_remove: Optional[Callable] = None):
        self.hooks_dict_ref = weakref.ref(hooks_dict) if not isinstance(hooks_dict, dict) else (lambda d=hooks_dict: d)
        self.id = RemovableHandle._next_id
        RemovableHandle._next_id += 1
        self.on_remove = on_remove

    def remove(self):
        """unregister"""
        d = self.hooks_dict_ref()
        if d is not None and self.id in d:
            del d[self.id]
        if self.on_remove:
            self.on_remove()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.remove()


class MethodWithHooks:
    """callable replacing a bound method; runs pre hooks, the method, post hooks"""

    def __init__(self, obj, attr: str):
        self.obj = obj
        self.attr = attr
        self.orig = getattr(type(obj), attr)
        self.pre_hooks: Dict[int, Callable] = {}
        self.post_hooks: Dict[int, Callable] = {}

    @classmethod
    def get(cls, obj, attr: str) -> "MethodWithHooks":
        """existing or new wrapper installed on obj"""
        cur = obj.__dict__.get(attr) if hasattr(obj, "__dict__") else None
        if isinstance(cur, MethodWithHooks):
            return cur
        m = cls(obj, attr)
        setattr(obj, attr, m)
        return m

    def _maybe_uninstall(self):
        if not self.pre_hooks and not self.post_hooks and self.obj.__dict__.get(self.attr) is self:
            delattr(self.obj, self.attr)

    def __call__(self, *args, **kwargs):
        for h in list(self.pre_hooks.values()):
            res = h(self.obj, args, kwargs)
            if res is not None:
                args, kwargs = res
        out = self.orig(self.obj, *args, **kwargs)
        for h in list(self.post_hooks.values()):
            res = h(self.obj, args, kwargs, out)
            if res is not None:
                out = res
        return out


def setup_pre_hook_on_method(obj, attr: str, hook: Callable[[Any, Tuple, Dict], Optional[Tuple[Tuple, Dict]]], *, prepend: bool = False) -> RemovableHandle:
    """hook(obj, args, kwargs) -> None | (args, kwargs), called before obj.attr(...)"""
    m = MethodWithHooks.get(obj, attr)
    h = RemovableHandle(m.pre_hooks, on_remove=m._maybe_uninstall)
    if prepend:
        items = {h.id: hook}
        items.update(m.pre_hooks)
        m.pre_hooks.clear()
        m.pre_hooks.update(items)
    else:
        m.pre_hooks[h.id] = hook
    return h


def setup_post_hook_on_method(obj, attr: str, hook: Callable, *, prepend: bool = False) -> RemovableHandle:
    """hook(obj, args, kwargs, result) -> None | new result, called after obj.attr(...)"""
    m = MethodWithHooks.get(obj, attr)
    h = RemovableHandle(m.post_hooks, on_remove=m._maybe_uninstall)
    m.post_hooks[h.id] = hook
    return h
