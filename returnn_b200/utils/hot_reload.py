"""
Hot reloading of user code referenced from the config: when a step function or model definition fails (or on request),
the modules that define the config's functions and classes are reloaded from disk and the config entries re-bound, so an
interactive session can fix the code and retry without restarting (and without reloading data and model).

Parity: returnn/util/hot_reload.py (should_use_hot_reloading :17, ConfigHotReloader :30, hot_reload_config :126).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Set, Tuple
import importlib
import os
import sys
import types


def should_use_hot_reloading(*, config=None) -> bool:
    """interactive terminal and ``use_hot_reloading`` in the config or ``RETURNN_USE_HOT_RELOADING=1``"""
    if not sys.stdin.isatty():
        return False
    if config is None:
        from ..config import get_global_config

        config = get_global_config(raise_exception=False)
    if config is not None and config.bool("use_hot_reloading", False):
        return True
    return os.environ.get("RETURNN_USE_HOT_RELOADING", "0") == "1"


def _is_custom_module(mod_name: Optional[str]) -> bool:
    """user code: not builtin, not this framework, not site-packages"""
    if not mod_name or mod_name in ("builtins", "__main__") or mod_name.split(".")[0] in ("returnn_b200", "torch", "numpy"):
        return False
    mod = sys.modules.get(mod_name)
    f = getattr(mod, "__file__", None)
    return bool(f) and "site-packages" not in f and not f.startswith(sys.prefix + "/lib")


def _walk(value: Any, *, visit: Callable[[Any], Optional[Any]], update: Optional[Callable[[Any], None]] = None, _seen: Optional[Set[int]] = None):
    """call ``visit`` on functions/classes/partials inside nested containers; if it returns a replacement, write it back"""
    _seen = _seen if _seen is not None else set()
    if id(value) in _seen:
        return
    _seen.add(id(value))
    if isinstance(value, (types.FunctionType, type)):
        new = visit(value)
        if new is not None and update is not None:
            update(new)
    elif isinstance(value, dict):
        for k in list(value.keys()):
            _walk(value[k], visit=visit, update=lambda v, k=k: value.__setitem__(k, v), _seen=_seen)
    elif isinstance(value, list):
        for i in range(len(value)):
            _walk(value[i], visit=visit, update=lambda v, i=i: value.__setitem__(i, v), _seen=_seen)
    elif isinstance(value, tuple):
        items = list(value)
        changed = []
        for i in range(len(items)):
            _walk(items[i], visit=visit, update=lambda v, i=i: (items.__setitem__(i, v), changed.append(1)), _seen=_seen)
        if changed and update is not None:
            update(tuple(items))
    elif hasattr(value, "func") and hasattr(value, "args") and hasattr(value, "keywords"):  # functools.partial
        import functools

        parts = {"func": value.func}
        _walk(value.func, visit=visit, update=lambda v: parts.__setitem__("func", v), _seen=_seen)
        if parts["func"] is not value.func and update is not None:
            update(functools.partial(parts["func"], *value.args, **(value.keywords or {})))


def _find_modules_in_config(config: Dict[str, Any]) -> Tuple[List[str], List[str], Dict[str, Set[str]]]:
    modules: List[str] = []
    keys: List[str] = []
    keys_per_module: Dict[str, Set[str]] = {}
    for k, v in config.items():
        found: List[str] = []

        def visit(obj, found=found):
            m = getattr(obj, "__module__", None)
            if _is_custom_module(m):
                found.append(m)
            return None

        _walk(v, visit=visit)
        if found:
            keys.append(k)
            for m in found:
                if m not in modules:
                    modules.append(m)
                keys_per_module.setdefault(m, set()).add(k)
    return modules, keys, keys_per_module


def _rebind(obj):
    """the object of the same qualified name in the (reloaded) module"""
    m = sys.modules.get(getattr(obj, "__module__", None) or "")
    if m is None or not _is_custom_module(m.__name__):
        return None
    cur: Any = m
    for part in getattr(obj, "__qualname__", obj.__name__).split("."):
        if part == "<locals>":
            return None
        cur = getattr(cur, part, None)
        if cur is None:
            return None
    return cur if cur is not obj else None


class ConfigHotReloader:
    """tracks the modification times of the user modules behind a config dict"""

    def __init__(self, config: Dict[str, Any]):
        self.config = config
        self._modules, self._keys, self._keys_per_module = _find_modules_in_config(config)
        self._mtimes = {m: os.path.getmtime(sys.modules[m].__file__) for m in self._modules}

    @property
    def modules(self) -> List[str]:
        """user modules referenced from the config"""
        return self._modules

    def any_module_changed(self) -> bool:
        """a source file is newer than at the last (re)load"""
        return any(os.path.getmtime(sys.modules[m].__file__) != t for m, t in self._mtimes.items())

    def reload_changed_modules(self):
        """reload and re-bind the config entries that point into the reloaded modules"""
        touched: Set[str] = set()
        for m in self._modules:
            t = os.path.getmtime(sys.modules[m].__file__)
            if t != self._mtimes[m]:
                print("Module %r has changed, reloading..." % m)
                importlib.reload(sys.modules[m])
                self._mtimes[m] = t
                touched |= self._keys_per_module[m]
        for k in self._keys:
            if k in touched:
                print("Updating config key %r..." % k)
                _walk(self.config[k], visit=_rebind, update=lambda v, k=k: self.config.__setitem__(k, v))

    def user_interaction(self, *, return_actions: Optional[Dict[str, str]] = None, shell_locals=None, shell_globals=None) -> str:
        """prompt: reload / retry or continue / debug / reraise / shell / quit; :return: the chosen return action key"""
        from .debug import debug_shell

        exc_type, exc, tb = sys.exc_info()
        assert sys.stdin.isatty()
        if return_actions is None:
            return_actions = {"t": "try again"} if exc is not None else {"c": "continue"}
        frame = sys._getframe(1)
        shell_locals = frame.f_locals if shell_locals is None else shell_locals
        shell_globals = frame.f_globals if shell_globals is None else shell_globals
        while True:
            choices = {"r": "reload modules", **return_actions}
            if exc is not None:
                choices.update({"d": "debug", "e": "reraise"})
            choices.update({"s": "shell", "q": "quit"})
            answer = input("Hot reloading: " + ", ".join("%r to %s" % kv for kv in choices.items()) + ": ").strip()
            if answer == "r":
                if self.any_module_changed():
                    self.reload_changed_modules()
                else:
                    print("No changes detected in", self._modules)
            elif answer in return_actions:
                return answer
            elif answer == "d" and exc is not None:
                debug_shell(dict(shell_locals, __traceback__=tb), shell_globals, exit_afterwards=False)
            elif answer == "e" and exc is not None:
                raise exc.with_traceback(tb)
            elif answer == "s":
                debug_shell(shell_locals, shell_globals, exit_afterwards=False)
            elif answer == "q":
                sys.exit(1)
            else:
                print("Invalid choice %r" % answer)


def hot_reload_config(config: Dict[str, Any]):
    """reload every user module behind the config and re-bind all entries"""
    modules, keys, _ = _find_modules_in_config(config)
    for m in modules:
        print("Reloading module %r..." % m)
        importlib.reload(sys.modules[m])
    for k in keys:
        _walk(config[k], visit=_rebind, update=lambda v, k=k: config.__setitem__(k, v))


_active: Optional[ConfigHotReloader] = None


def enable(config) -> Optional[ConfigHotReloader]:
    """track the user modules behind ``config`` (a :class:`Config`); the engine asks :func:`get_active` when a step fails"""
    global _active
    if not should_use_hot_reloading(config=config):
        return None
    _active = ConfigHotReloader(config.typed_dict)
    return _active


def get_active() -> Optional[ConfigHotReloader]:
    """the reloader installed by :func:`enable`, if any"""
    return _active
