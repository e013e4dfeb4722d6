"""
Configuration object.

Three file formats: Python (``#!`` first line or ``.py`` suffix; executed, every global becomes a typed entry),
JSON (starts with ``{``) and the line format ``key value[,value...]`` with ``#`` comments.
Command line: short/long options for a handful of common keys, ``--config file``, and ``++key value`` pairs.
Entries from Python/JSON live in ``typed_dict`` (native Python types); entries from the line format and the
command line live in ``dict`` as lists of strings and are coerced by the accessor used.

Parity: returnn/config.py (Config :22, load_file :99-162, parse_cmd_args :177, accessors :341-636,
get_global_config :665, SubProcCopyGlobalConfigPreInitFunc :818).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Type, TypeVar, Union
import builtins
import contextlib
import os
import sys
import time
import types as _types

__all__ = [
    "Config",
    "set_global_config",
    "get_global_config",
    "global_config_ctx",
    "network_json_from_config",
    "SubProcCopyGlobalConfigPreInitFunc",
]

T = TypeVar("T")
_PyModuleName = "__returnn_config__"

# (short, long/dest) command line options that map 1:1 onto a config key
_CMD_OPTS: List[Tuple[str, str, str]] = [
    ("-a", "--activation", "activation"),
    ("-b", "--batch_size", "batch_size"),
    ("-c", "--chunking", "chunking"),
    ("-d", "--description", "description"),
    ("-e", "--epoch", "epoch"),
    ("-E", "--eval", "eval"),
    ("-i", "--save_interval", "save_interval"),
    ("-j", "--dropout", "dropout"),
    ("-k", "--output_file", "output_file"),
    ("-l", "--log", "log"),
    ("-L", "--load", "load"),
    ("-m", "--momentum", "momentum"),
    ("-n", "--num_epochs", "num_epochs"),
    ("-o", "--order", "order"),
    ("-q", "--cache", "cache"),
    ("-r", "--learning_rate", "learning_rate"),
    ("-t", "--truncate", "truncate"),
    ("-u", "--device", "device"),
    ("-v", "--verbose", "log_verbosity"),
    ("-w", "--window", "window"),
    ("-x", "--task", "task"),
    ("-z", "--max_sequences", "max_seqs"),
]


class Config:
    """
    Key/value store with typed and string-list entries.
    """

    def __init__(self, items: Optional[Dict[str, Any]] = None):
        self.dict: Dict[str, List[str]] = {}
        self.typed_dict: Dict[str, Any] = {}
        self.network_topology_json: Optional[str] = None
        self.files: List[str] = []
        if items is not None:
            self.typed_dict.update(items)

    # -- pickling: functions/modules/classes defined inside the config cannot be pickled by reference
    # to an importable module, so the state carries the source files and is re-executed on the other side.
    def __getstate__(self):
        import io
        import pickle

        state = {"dict": self.dict, "files": self.files, "network_topology_json": self.network_topology_json}
        simple, by_file = {}, []
        for k, v in self.typed_dict.items():
            if k in ("config", "__builtins__", "__file__", "__name__", "__package__"):
                continue
            try:
                buf = io.BytesIO()
                pickle.Pickler(buf).dump(v)
                simple[k] = v
            except Exception:
                by_file.append(k)
        state["typed_simple"] = simple
        state["typed_by_file"] = by_file
        return state

    def __setstate__(self, state):
        self.dict = state["dict"]
        self.files = []
        self.typed_dict = {}
        self.network_topology_json = state["network_topology_json"]
        if state["typed_by_file"]:
            for f in state["files"]:
                if os.path.isfile(f) and self.get_config_file_type(f) == "py":
                    self.load_file(f)
        self.files = state["files"]
        self.typed_dict.update(state["typed_simple"])

    def load_file(self, f):
        """
        Read a config file (path or stream) in any of the three formats and merge it.
        """
        if isinstance(f, str):
            assert os.path.isfile(f), "config file not found: %r" % f
            self.files.append(f)
            filename = f
            content = open(filename).read()
        else:
            filename = "<config string>"
            content = f.read()
        content = content.strip()
        if content.startswith("#!") or filename.endswith(".py"):
            from .utils.basic import custom_exec

            user_ns = self.typed_dict
            user_ns.update({"config": self, "__file__": filename, "__name__": _PyModuleName})
            custom_exec(content, filename, user_ns, user_ns)
            _install_config_module_proxy()
            return
        if content.startswith("{"):
            from .utils.basic import load_json

            json_content = load_json(content=content)
            assert isinstance(json_content, dict)
            self.update(json_content)
            return
        for line in content.splitlines():
            if "#" in line:
                line = line[: line.index("#")]
            line = line.strip()
            if not line:
                continue
            parts = line.split(None, 1)
            assert len(parts) == 2, "unable to parse config line: %r" % line
            self.add_line(key=parts[0], value=parts[1])

    @classmethod
    def get_config_file_type(cls, f: str) -> str:
        """:return: "py", "js" or "txt" """
        with open(f, "r") as fh:
            start = fh.read(3)
        if start.startswith("#!") or f.endswith(".py"):
            return "py"
        if start.startswith("{"):
            return "js"
        return "txt"

    def parse_cmd_args(self, args: Sequence[str]):
        """
        :param args: command line without the standalone config file names
        """
        import argparse

        parser = argparse.ArgumentParser(
            usage="%(prog)s [config_filename]* [option]* [++key value]*", add_help=True, allow_abbrev=False
        )
        for short, long_, dest in _CMD_OPTS:
            parser.add_argument(short, long_, dest=dest, default=None)
        parser.add_argument("-V", "--version", action="store_true", dest="version")
        parser.add_argument("--config", dest="load_config", default=None)
        options, rest = parser.parse_known_args(list(args))
        if options.version:
            from . import __long_version__

            print(
                "returnn_b200 version %s, date/time %s, pid %i, cwd %s, Python %s"
                % (__long_version__, time.strftime("%Y-%m-%d-%H-%M-%S (UTC%z)"), os.getpid(), os.getcwd(), sys.executable)
            )
            sys.exit(0)
        for opt, val in vars(options).items():
            if val is None or opt == "version":
                continue
            if opt == "load_config":
                self.load_file(val)
            else:
                self.add_line(opt, val)
        assert len(rest) % 2 == 0, "expect (++key, value) config tuples in remaining args: %r" % (rest,)
        for i in range(0, len(rest), 2):
            key, value = rest[i : i + 2]
            assert key.startswith("++"), "expect key prefixed with '++' in (%r, %r)" % (key, value)
            if value[:2] == "+-":
                value = value[1:]
            self.add_line(key=key[2:], value=value)

    def add_line(self, key: str, value: str):
        """
        Add one (key, string value) pair. A key that already has a typed value keeps its type
        (the string is evaluated as a Python expression unless the previous value was a str).
        """
        if key in self.typed_dict:
            value_type = type(self.typed_dict[key])
            if value_type is not str:
                try:
                    value = eval(value)
                except (SyntaxError, NameError):
                    print(
                        "WARNING: can't evaluate config param %r to previous type: %s. Keeping as string."
                        % (value, value_type),
                        file=sys.stderr,
                    )
            self.typed_dict[key] = value
            return
        if value.find(",") > 0:
            values = value.split(",")
        else:
            values = [value]
        if key == "include":
            for f in values:
                self.load_file(f)
        else:
            self.dict[key] = values

    def has(self, key: str) -> builtins.bool:
        """key present in either store"""
        return key in self.typed_dict or key in self.dict

    def is_typed(self, key: str) -> builtins.bool:
        """key has a typed value"""
        return key in self.typed_dict

    def is_true(self, key: str, default: builtins.bool = False) -> builtins.bool:
        """typed truth value or parsed bool"""
        if self.is_typed(key):
            return builtins.bool(self.typed_dict[key])
        return self.bool(key, default=default)

    def is_of_type(self, key: str, types) -> builtins.bool:
        """typed and isinstance"""
        if key in self.typed_dict:
            return isinstance(self.typed_dict[key], types)
        return False

    def get_of_type(self, key: str, types, default=None):
        """typed value if isinstance else default"""
        if key in self.typed_dict and isinstance(self.typed_dict[key], types):
            return self.typed_dict[key]
        return default

    def set(self, key: str, value: Any):
        """set typed value"""
        self.typed_dict[key] = value
        self.dict.pop(key, None)

    def update(self, dikt: Dict[str, Any]):
        """set many"""
        for k, v in dikt.items():
            self.set(k, v)

    def value(self, key: str, default: T, index: Optional[builtins.int] = None, list_join_str: str = ",") -> Union[str, T]:
        """string view of an entry"""
        if key in self.typed_dict:
            ls = self.typed_dict[key]
            if index is None:
                if isinstance(ls, (list, tuple)):
                    return list_join_str.join(str(v) for v in ls)
                if ls is None:
                    return default
                return str(ls)
            if isinstance(ls, (list, tuple)):
                return str(ls[index])
            return str(ls)
        if key in self.dict:
            ls = self.dict[key]
            if index is None:
                return list_join_str.join(ls)
            if index < len(ls):
                return ls[index]
        return default

    def typed_value(self, key: str, default: Optional[T] = None, index: Optional[builtins.int] = None):
        """typed value, falling back to the string list entry (joined / indexed)"""
        value = self.typed_dict.get(key, None)
        if value is None and key not in self.typed_dict:
            if key in self.dict:
                ls = self.dict[key]
                value = (ls[0] if len(ls) == 1 else ls) if index is None else ls[index]
            else:
                return default
        elif index is not None and isinstance(value, (tuple, list)):
            value = value[index]
        if value is None:
            return default
        return value

    def opt_typed_value(self, key: str, default: Optional[T] = None):
        """typed value or string value"""
        if key in self.typed_dict:
            return self.typed_dict[key]
        return self.value(key, default)

    def int(self, key: str, default: T, index: builtins.int = 0) -> Union[builtins.int, T]:
        """int view"""
        if key in self.typed_dict:
            value = self.typed_value(key, default=default, index=index)
            if value is not None:
                assert isinstance(value, builtins.int), "config key %r: expected int, got %r" % (key, value)
            return value
        if key in self.dict:
            return builtins.int(self.value(key, default, index))
        return default

    def bool(self, key: str, default: T, index: builtins.int = 0) -> Union[builtins.bool, T]:
        """bool view"""
        if key in self.typed_dict:
            value = self.typed_value(key, default=default, index=index)
            if isinstance(value, builtins.int):
                value = builtins.bool(value)
            if value is not None:
                assert isinstance(value, builtins.bool), "config key %r: expected bool, got %r" % (key, value)
            return value
        if key not in self.dict:
            return default
        from .utils.basic import to_bool

        return to_bool(self.value(key, None, index))

    def bool_or_other(self, key: str, default: T = None, index: builtins.int = 0):
        """bool if it parses as one, else the raw value"""
        if key in self.typed_dict:
            return self.typed_value(key, default=default, index=index)
        if key not in self.dict:
            return default
        v = self.value(key, default=None, index=index)
        from .utils.basic import to_bool

        try:
            return to_bool(v)
        except ValueError:
            return v

    def float(self, key: str, default: T, index: builtins.int = 0) -> Union[builtins.float, T]:
        """float view"""
        if key in self.typed_dict:
            value = self.typed_value(key, default=default, index=index)
        else:
            value = self.value(key, default, index)
        if value is not None:
            if isinstance(value, str):
                assert value.lower() != "none"
                return builtins.float(value)
            assert isinstance(value, (builtins.int, builtins.float)), "config key %r: expected float" % key
        return value

    def list(self, key: str, default: Optional[T] = None) -> Union[List[str], T]:
        """list view"""
        if default is None:
            default = []
        if key in self.typed_dict:
            value = self.typed_value(key, default=default)
            if value is None:
                return default
            if not isinstance(value, (tuple, builtins.list)):
                value = [value]
            return builtins.list(value)
        if key not in self.dict:
            return default
        return builtins.list(self.dict[key])

    def int_list(self, key: str, default=None):
        """list of int"""
        if default is None:
            default = []
        if key in self.typed_dict:
            value = self.typed_value(key, default=default)
            if value is None:
                return default
            if not isinstance(value, (tuple, builtins.list)):
                value = [value]
            for x in value:
                assert isinstance(x, builtins.int)
            return builtins.list(value)
        return [builtins.int(x) for x in self.list(key, default)]

    def float_list(self, key: str, default=None):
        """list of float"""
        if default is None:
            default = []
        if key in self.typed_dict:
            value = self.typed_value(key, default=default)
            if value is None:
                return default
            if not isinstance(value, (tuple, builtins.list)):
                value = [value]
            return [builtins.float(x) for x in value]
        return [builtins.float(x) for x in self.list(key, default)]

    def int_pair(self, key: str, default: Optional[Tuple[builtins.int, builtins.int]] = None):
        """(a, b) from "a:b" / "a" / typed tuple"""
        if default is None:
            default = (0, 0)
        if not self.has(key):
            return default
        if key in self.typed_dict:
            value = self.typed_value(key, default=default)
            if not isinstance(value, (tuple, builtins.list)):
                value = (value, value)
            assert len(value) == 2
            return builtins.int(value[0]), builtins.int(value[1])
        value = self.value(key, "")
        if ":" in value:
            a, b = value.split(":")
            return builtins.int(a), builtins.int(b)
        return builtins.int(value), builtins.int(value)

    def __repr__(self):
        return "<Config files=%r>" % (self.files,)


_global_config: Optional[Config] = None


def set_global_config(config: Optional[Config]):
    """set the process-wide config"""
    global _global_config
    _global_config = config
    _install_config_module_proxy()


def get_global_config(*, raise_exception: bool = True, auto_create: bool = False, return_empty_if_none: bool = False):
    """
    :return: the process-wide config
    """
    global _global_config
    if _global_config is not None:
        return _global_config
    if auto_create:
        config = Config()
        set_global_config(config)
        return config
    if return_empty_if_none:
        return Config()
    if raise_exception:
        raise Exception("No global config found.")
    return None


@contextlib.contextmanager
def global_config_ctx(config: Config):
    """temporarily replace the global config"""
    global _global_config
    prev = _global_config
    try:
        set_global_config(config)
        yield
    finally:
        _global_config = prev


def network_json_from_config(config: Config):
    """the net-dict of legacy configs (kept for tools that only read it)"""
    if config.has("network") and config.is_typed("network"):
        return config.typed_value("network")
    return None


class _ConfigModuleProxy(_types.ModuleType):
    """``import __returnn_config__`` gives attribute access to the global config's typed entries."""

    def __getattr__(self, item):
        cfg = _global_config
        if cfg is None or item not in cfg.typed_dict:
            raise AttributeError(item)
        return cfg.typed_dict[item]

    def __dir__(self):
        cfg = _global_config
        return sorted(cfg.typed_dict.keys()) if cfg else []


def _install_config_module_proxy():
    if _PyModuleName not in sys.modules:
        sys.modules[_PyModuleName] = _ConfigModuleProxy(_PyModuleName)


class SubProcCopyGlobalConfigPreInitFunc:
    """
    Picklable callable handed to worker processes (spawn): carries the parent's global config and installs it
    (and the better exception hook) in the child before anything else runs.
    """

    def __init__(self):
        self.global_config = get_global_config(raise_exception=False)

    def __call__(self):
        from .utils import better_exchook

        better_exchook.install()
        if self.global_config is not None:
            set_global_config(self.global_config)
