"""
Construct modules from ``{"class": "rf.Linear", ...}`` dicts.  Parity: returnn/frontend/build_from_dict.py.
"""

from __future__ import annotations
from typing import Any, Dict, Type, TypeVar, Union
import importlib

__all__ = ["build_from_dict", "build_dict"]
T = TypeVar("T")


def _resolve(name: str):
    if name.startswith("rf."):
        from .. import frontend as rf

        obj: Any = rf
        for part in name[3:].split("."):
            obj = getattr(obj, part)
        return obj
    if "." in name:
        mod_name, attr = name.rsplit(".", 1)
        if mod_name.startswith("returnn."):
            mod_name = "returnn_b200." + mod_name[len("returnn."):].replace("util.", "utils.")
        try:
            return getattr(importlib.import_module(mod_name), attr)
        except ImportError:
            # nested attribute path
            parts = name.split(".")
            for i in range(len(parts) - 1, 0, -1):
                try:
                    obj = importlib.import_module(".".join(parts[:i]))
                except ImportError:
                    continue
                for p in parts[i:]:
                    obj = getattr(obj, p)
                return obj
            raise
    raise ValueError("build_from_dict: cannot resolve class %r (use 'rf.<Name>' or a dotted path)" % name)


def build_from_dict(d: Dict[str, Any], *args, **kwargs):
    """``d["class"]`` (str or class) called with the remaining items + args/kwargs"""
    if not isinstance(d, dict):
        raise TypeError("build_from_dict: expected dict, got %r" % type(d))
    d = dict(d)
    cls = d.pop("class", None)
    if cls is None:
        raise ValueError("build_from_dict: missing 'class' in %r" % d)
    if isinstance(cls, str):
        cls = _resolve(cls)
    d.update(kwargs)
    return cls(*args, **d)


def build_dict(cls: Union[type, Any], **kwargs) -> Dict[str, Any]:
    """inverse: dict which build_from_dict turns into cls(**kwargs)"""
    name = "%s.%s" % (cls.__module__, cls.__qualname__)
    if name.startswith("returnn_b200.frontend."):
        from .. import frontend as rf

        if getattr(rf, cls.__qualname__, None) is cls:  # the short form only for what the package namespace exports
            name = "rf." + cls.__qualname__
    return {"class": name, **kwargs}
