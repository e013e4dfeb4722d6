"""
``rf.Module``: base class of all models and layers. Parameters and sub-modules are plain attributes;
the attribute path is the name in the checkpoint.

Parity: returnn/frontend/module.py:17.
"""

from __future__ import annotations
from typing import Any, Dict, Iterator, List, Optional, Set, Tuple, Union
import copy as _copy
from ..tensor import Tensor, Dim

__all__ = ["Module", "Functional"]


class Module:
    """
    Base class. Subclasses define ``__init__`` (creating :class:`rf.Parameter` and sub-modules as attributes)
    and ``__call__``.
    """

    _is_initialized = False

    def __init__(self):
        pass

    def __repr__(self):
        return "<%s>" % self.__class__.__qualname__

    def default_initial_state(self, *, batch_dims):
        """initial recurrent state; None for stateless modules"""
        state = None
        from .state import State

        for key, mod in self.named_children():
            sub = mod.default_initial_state(batch_dims=batch_dims)
            if sub:
                if state is None:
                    state = State()
                state[key] = sub
        return state

    def get_default_name(self) -> str:
        """name from the class name"""
        name = self.__class__.__name__
        return name[:1].lower() + name[1:]

    def __call__(self, *args, **kwargs):
        raise NotImplementedError("%s.__call__" % self.__class__.__name__)

    def get_deep(self, target: str) -> Any:
        """a.b.c attribute lookup"""
        if not target:
            return self
        obj: Any = self
        for part in target.split("."):
            obj = obj[int(part)] if part.isdigit() and hasattr(obj, "__getitem__") and not hasattr(obj, part) else getattr(obj, part)
        return obj

    def set_deep(self, target: str, value: Any) -> None:
        """a.b.c = value"""
        if "." in target:
            prefix, target = target.rsplit(".", 1)
            mod = self.get_deep(prefix)
        else:
            mod = self
        setattr(mod, target, value)

    def children(self) -> Iterator["Module"]:
        """direct sub-modules"""
        return (m for _, m in self.named_children())

    def named_children(self) -> Iterator[Tuple[str, "Module"]]:
        """direct (name, sub-module) pairs"""
        seen: Set[int] = set()
        for name, value in vars(self).items():
            if isinstance(value, Module) and id(value) not in seen:
                seen.add(id(value))
                yield name, value

    def modules(self) -> Iterator["Module"]:
        """self and all nested sub-modules"""
        return (m for _, m in self.named_modules())

    def named_modules(self, memo: Optional[Set[int]] = None, prefix: str = "") -> Iterator[Tuple[str, "Module"]]:
        """(path, module) for self and all nested"""
        if memo is None:
            memo = set()
        if id(self) in memo:
            return
        memo.add(id(self))
        yield prefix, self
        for name, mod in self.named_children():
            yield from mod.named_modules(memo=memo, prefix=(prefix + "." if prefix else "") + name)

    def named_parameters(self, *, recurse: bool = True) -> Iterator[Tuple[str, "Parameter"]]:
        """(path, parameter), each parameter once"""
        from .parameter import Parameter

        memo: Set[int] = set()
        mods = self.named_modules() if recurse else [("", self)]
        for prefix, mod in mods:
            for name, value in vars(mod).items():
                if isinstance(value, Parameter) and id(value) not in memo:
                    memo.add(id(value))
                    yield (prefix + "." if prefix else "") + name, value

    def parameters(self, *, recurse: bool = True) -> Iterator["Parameter"]:
        """all parameters"""
        return (p for _, p in self.named_parameters(recurse=recurse))

    @property
    def has_parameters(self) -> bool:
        """any parameter at all"""
        for _ in self.parameters():
            return True
        return False

    def apply(self, fn) -> "Module":
        """fn(module) for all modules, children first"""
        for child in self.children():
            child.apply(fn)
        fn(self)
        return self

    def to(self, *, device: Optional[str] = None, dtype: Optional[str] = None):
        """move / cast all parameters in place"""
        import torch
        from ._utils import torch_dtype

        for p in self.parameters():
            raw = p._raw_tensor
            kw = {}
            if device is not None:
                kw["device"] = device
            if dtype is not None and raw.is_floating_point():
                kw["dtype"] = torch_dtype(dtype)
                p.dtype = dtype
            with torch.no_grad():
                new = raw.data.to(**kw)
            if isinstance(raw, torch.nn.Parameter):
                raw.data = new
            else:
                p._raw_tensor = new
        return self

    def __getstate__(self):
        return self.__dict__

    def __setstate__(self, state):
        self.__dict__.update(state)


class Functional(Module):
    """wraps a function as a module (for Sequential)"""

    def __init__(self, func):
        super().__init__()
        assert callable(func)
        self.func = func

    def __repr__(self):
        return "%s(%s)" % (self.__class__.__name__, getattr(self.func, "__qualname__", self.func))

    def get_default_name(self) -> str:
        """function name"""
        return getattr(self.func, "__qualname__", "func")

    def __call__(self, *args, **kwargs):
        return self.func(*args, **kwargs)
