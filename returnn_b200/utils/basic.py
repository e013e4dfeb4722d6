"""
Generic helpers shared by all layers: sentinels, behavior version, ``NumbersDict``, option-dict checking,
running statistics, time / size formatting, file locks, BLEU, and small process/environment helpers.

Parity: returnn/util/basic.py (BackendEngine :147-206, BehaviorVersion :238-368, NumbersDict :1903,
CollectionReadCheckCovered :2781, Stats :4042, should_write_to_disk :3850-3873).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, TypeVar, Union
import builtins
import collections
import contextlib
import math
import os
import sys
import time
import json
import re
import numpy

T = TypeVar("T")


class NotSpecified:
    """Sentinel type for "argument not given" where ``None`` is a valid value."""

    @classmethod
    def resolve(cls, value, default):
        """:return: default if value is NotSpecified else value"""
        return default if value is NotSpecified else value

    def __new__(cls, *args, **kwargs):
        raise TypeError("NotSpecified is a sentinel, not to be instantiated")


class Entity:
    """Named unique object, e.g. for markers like ``single_step_dim``-style sentinels."""

    def __init__(self, name: Optional[str] = None, *, global_base=None, global_name: Optional[str] = None):
        self.name = name
        self.global_base = global_base
        self.global_name = global_name

    def __repr__(self):
        return "<%s>" % (self.name or "entity")

    def __reduce__(self):
        if self.global_name:
            if self.global_base is not None:
                return getattr, (self.global_base, self.global_name)
            return self.global_name
        raise Exception("cannot pickle Entity %r" % self)

    def __getstate__(self):
        if self.global_name:
            raise Exception("pickle by global name")
        return self.__dict__


class OptionalNotImplementedError(NotImplementedError):
    """Raised by optional API functions which a subclass may leave out."""


class BackendEngine:
    """
    Which engine runs the model. This framework has exactly one: torch on B200.
    The enum keeps the reference's names so that configs with ``backend = "torch"`` validate.
    """

    Torch = 3
    selected_engine: Optional[int] = None

    @classmethod
    def select_engine(cls, *, engine=None, default_fallback_engine=None, config=None, _select_rf_backend=True):
        """Select by config key ``backend`` (only "torch" is accepted)."""
        if engine is None:
            backend = None
            if config is not None:
                backend = config.value("backend", None)
            if backend not in (None, "torch", "pytorch"):
                raise ValueError(
                    "backend %r: this framework is torch-only (no TF / JAX engines); use backend='torch'" % backend
                )
            engine = cls.Torch
        cls.selected_engine = engine

    @classmethod
    def get_selected_engine(cls) -> int:
        """:return: engine id (always Torch)"""
        if cls.selected_engine is None:
            cls.selected_engine = cls.Torch
        return cls.selected_engine

    @classmethod
    def is_torch_selected(cls) -> bool:
        """always true once selected"""
        return cls.get_selected_engine() == cls.Torch

    @classmethod
    def is_tensorflow_selected(cls) -> bool:
        """never"""
        return False

    @classmethod
    def is_jax_selected(cls) -> bool:
        """never"""
        return False


class BehaviorVersion:
    """
    Global ``behavior_version``. Gates changed defaults. Latest known version is 30.
    """

    _latest_behavior_version = 30
    _behavior_version: Optional[int] = None
    _min_behavior_version: int = 0

    class RequirementNotSatisfied(Exception):
        """the config does something that the selected behavior version forbids"""

    @classmethod
    def set(cls, version: Optional[int]):
        """set once; setting the same value again is fine"""
        if version == cls._behavior_version:
            return
        if cls._behavior_version is not None:
            raise Exception(f"behavior_version already set to {cls._behavior_version}, cannot reset to {version}")
        assert version >= cls._min_behavior_version, "behavior_version %i < required minimum %i" % (
            version,
            cls._min_behavior_version,
        )
        if version > cls._latest_behavior_version:
            print(
                "Warning: behavior_version %i > latest known %i" % (version, cls._latest_behavior_version),
                file=sys.stderr,
            )
        cls._behavior_version = version

    @classmethod
    def get(cls) -> int:
        """current version, or the minimum if unset"""
        if cls._behavior_version is not None:
            return cls._behavior_version
        return cls._min_behavior_version

    @classmethod
    def get_if_set(cls) -> Optional[int]:
        """current version or None"""
        return cls._behavior_version

    @classmethod
    def set_min_behavior_version(cls, min_behavior_version: int):
        """some features need a minimum behavior version"""
        if min_behavior_version < cls._min_behavior_version:
            return
        assert min_behavior_version <= cls._latest_behavior_version
        if cls._behavior_version is not None and cls._behavior_version < min_behavior_version:
            raise cls.RequirementNotSatisfied(
                f"require min behavior_version {min_behavior_version}, have {cls._behavior_version}"
            )
        cls._min_behavior_version = min_behavior_version

    @classmethod
    def is_set(cls) -> bool:
        """whether explicitly set"""
        return cls._behavior_version is not None

    @classmethod
    def require(cls, condition: bool, message: str, version: int):
        """raise if ``not condition`` and behavior_version >= version"""
        assert version <= cls._latest_behavior_version
        if not condition and cls.get() >= version:
            raise cls.RequirementNotSatisfied(
                "%s (required since behavior_version >= %i, current %i)" % (message, version, cls.get())
            )

    @classmethod
    def _reset(cls, version: Optional[int] = None, min_version: int = 0):
        """for tests"""
        cls._behavior_version = version
        cls._min_behavior_version = min_version


def get_fwd_compat_kwargs() -> Dict[str, Any]:
    """
    A kwarg with a random name passed to every user callable,
    so that user functions must accept ``**kwargs`` and stay forward compatible.
    """
    import random

    return {"__fwd_compat_random_arg_%03i" % random.randint(0, 999): None}


def get_login_username() -> str:
    """:return: user name, safe for paths"""
    try:
        import getpass

        return getpass.getuser()
    except Exception:
        return os.environ.get("USER", "user")


def get_hostname() -> str:
    """:return: short hostname"""
    import socket

    try:
        return socket.gethostname()
    except Exception:
        return "localhost"


def custom_exec(source: str, source_filename: str, user_ns: Dict[str, Any], user_global_ns: Dict[str, Any]):
    """compile + exec with a proper filename so that tracebacks show the config lines"""
    if not source.endswith("\n"):
        source += "\n"
    co = compile(source, source_filename, "exec")
    user_global_ns["__package__"] = user_global_ns.get("__package__") or None
    eval(co, user_global_ns, user_ns)


_json_comment_re = re.compile(r"^\s*#.*$", re.MULTILINE)


def load_json(filename: Optional[str] = None, content: Optional[str] = None) -> Dict[str, Any]:
    """JSON with ``#`` comment lines allowed"""
    if content is None:
        assert filename
        content = open(filename).read()
    content = _json_comment_re.sub("", content)
    try:
        return json.loads(content)
    except ValueError as e:
        raise Exception("config looks like JSON but invalid json content, %r" % e)


def hms(s: float) -> str:
    """seconds -> h:mm:ss"""
    s = int(s)
    m, s = divmod(s, 60)
    h, m = divmod(m, 60)
    return "%d:%02d:%02d" % (h, m, s)


def hms_fraction(s: float, decimals: int = 4) -> str:
    """seconds -> h:mm:ss.ffff"""
    s, frac = divmod(s, 1)
    s = int(s)
    m, s = divmod(s, 60)
    h, m = divmod(m, 60)
    return "%d:%02d:%02d.%s" % (h, m, s, ("%%.%if" % decimals % frac)[2:])


def human_size(n: float, factor: int = 1000, frac: float = 0.8, prec: int = 1) -> str:
    """number -> '1.2K' style"""
    postfixes = ["", "K", "M", "G", "T", "P"]
    i = 0
    while i < len(postfixes) - 1 and n > (factor ** (i + 1)) * frac:
        i += 1
    if i == 0:
        return str(n)
    return ("%." + str(prec) + "f") % (float(n) / (factor**i)) + postfixes[i]


def human_bytes_size(n: float, factor: int = 1024, frac: float = 0.8, prec: int = 1) -> str:
    """bytes -> '1.2GB' style"""
    return human_size(n, factor=factor, frac=frac, prec=prec) + "B"


def parse_human_size(s: str) -> int:
    """'4G' -> int"""
    s = s.strip()
    mult = {"K": 1024, "M": 1024**2, "G": 1024**3, "T": 1024**4}
    if s and s[-1].upper() == "B":
        s = s[:-1]
    if s and s[-1].upper() in mult:
        return int(float(s[:-1]) * mult[s[-1].upper()])
    return int(float(s))


def uniq(seq: Iterable[T]) -> List[T]:
    """consecutive duplicates removed"""
    out = []
    for x in seq:
        if not out or out[-1] != x:
            out.append(x)
    return out


def unique_list(seq: Iterable[T]) -> List[T]:
    """order-preserving unique"""
    seen = set()
    out = []
    for x in seq:
        if x not in seen:
            seen.add(x)
            out.append(x)
    return out


def make_seq_of_type(cls, seq):
    """convert seq to cls (tuple/list), keep namedtuples"""
    if hasattr(cls, "_fields"):
        return cls(*seq)
    return cls(seq)


def simple_obj_repr(obj) -> str:
    """ClassName(arg=value, ...) from ``__init__`` arg names"""
    import inspect

    names = [p for p in inspect.signature(obj.__class__.__init__).parameters if p != "self"]
    return obj.__class__.__name__ + "(%s)" % ", ".join("%s=%r" % (n, getattr(obj, n, None)) for n in names)


class CollectionReadCheckCovered:
    """
    Wraps an options dict and records which keys were read,
    so that leftover (unknown, probably misspelled) keys can be reported.
    """

    def __init__(self, collection: Dict[str, Any], truth_value: Optional[bool] = None):
        self.collection = collection
        self.got_items = set()
        self.truth_value = bool(collection) if truth_value is None else truth_value

    @classmethod
    def from_bool_or_dict(cls, value) -> "CollectionReadCheckCovered":
        """True/False/None/dict -> instance"""
        if isinstance(value, cls):
            return value
        if value is None or isinstance(value, bool):
            return cls(collection={}, truth_value=bool(value))
        if isinstance(value, dict):
            return cls(collection=value, truth_value=True)
        raise TypeError("invalid options value %r" % (value,))

    def __getitem__(self, item):
        res = self.collection[item]
        self.got_items.add(item)
        return res

    def get(self, item, default=None):
        """dict.get, recording the read"""
        if item in self.collection:
            return self[item]
        return default

    def __contains__(self, item):
        return item in self.collection

    def __bool__(self):
        return self.truth_value

    def __len__(self):
        return len(self.collection)

    def __iter__(self):
        for k in self.collection:
            yield self[k]

    def __repr__(self):
        return "%s(%r)" % (self.__class__.__name__, self.collection)

    def assert_all_read(self):
        """raise on keys never read"""
        remaining = set(self.collection).difference(self.got_items)
        assert not remaining, "The keys %r were not read in the collection %r." % (sorted(remaining), self.collection)


class NumbersDict:
    """
    Dict of numbers with element-wise arithmetic and a broadcast default value.
    Used for sequence lengths per data key (``{"data": 123, "classes": 17}``).
    """

    def __init__(self, auto_convert=None, numbers_dict=None, broadcast_value=None):
        if auto_convert is not None:
            assert numbers_dict is None and broadcast_value is None
            if isinstance(auto_convert, dict):
                numbers_dict = auto_convert
            elif isinstance(auto_convert, NumbersDict):
                numbers_dict = auto_convert.dict
                broadcast_value = auto_convert.value
            else:
                broadcast_value = auto_convert
        self.dict: Dict[str, Any] = dict(numbers_dict or {})
        self.value = broadcast_value
        self.max = self._max_error

    def copy(self) -> "NumbersDict":
        """copy"""
        return NumbersDict(self)

    @classmethod
    def constant_like(cls, const_number, numbers_dict: "NumbersDict") -> "NumbersDict":
        """same keys, constant value"""
        return NumbersDict(
            broadcast_value=const_number if numbers_dict.value is not None else None,
            numbers_dict={k: const_number for k in numbers_dict.dict},
        )

    def copy_like(self, numbers_dict: "NumbersDict") -> "NumbersDict":
        """self's values under numbers_dict's keys"""
        if self.value is not None:
            return NumbersDict(
                broadcast_value=self.value if numbers_dict.value is not None else None,
                numbers_dict={k: self[k] for k in numbers_dict.dict},
            )
        return NumbersDict(numbers_dict={k: self[k] for k in numbers_dict.dict})

    @property
    def keys_set(self):
        """set of keys"""
        return set(self.dict.keys())

    def __getitem__(self, key):
        if self.value is not None:
            return self.dict.get(key, self.value)
        return self.dict[key]

    def __setitem__(self, key, value):
        self.dict[key] = value

    def __delitem__(self, key):
        del self.dict[key]

    def __contains__(self, key):
        return key in self.dict

    def get(self, key, default=None):
        """dict.get with broadcast default"""
        return self.dict.get(key, default if self.value is None else self.value)

    def has_values(self) -> bool:
        """anything in here"""
        return bool(self.dict) or self.value is not None

    def unary_op(self, op: Callable) -> "NumbersDict":
        """apply op to every value"""
        res = NumbersDict()
        if self.value is not None:
            res.value = op(self.value)
        for k, v in self.dict.items():
            res.dict[k] = op(v)
        return res

    @classmethod
    def bin_op_scalar_optional(cls, self, other, zero, op):
        """op where None means missing"""
        if self is None and other is None:
            return None
        if self is None:
            self = zero
        if other is None:
            other = zero
        return op(self, other)

    @classmethod
    def bin_op(cls, self, other, op, zero, result=None) -> "NumbersDict":
        """element-wise op with key union"""
        if not isinstance(self, NumbersDict):
            if isinstance(other, NumbersDict):
                self = NumbersDict.constant_like(self, numbers_dict=other)
            else:
                self = NumbersDict(self)
        if not isinstance(other, NumbersDict):
            other = NumbersDict.constant_like(other, numbers_dict=self)
        if result is None:
            result = NumbersDict()
        assert isinstance(result, NumbersDict)
        for k in self.keys_set | other.keys_set:
            result[k] = cls.bin_op_scalar_optional(self.get(k, None), other.get(k, None), zero=zero, op=op)
        result.value = cls.bin_op_scalar_optional(self.value, other.value, zero=zero, op=op)
        return result

    def __add__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a + b, zero=0)

    __radd__ = __add__

    def __iadd__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a + b, zero=0, result=self)

    def __sub__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a - b, zero=0)

    def __rsub__(self, other):
        return self.bin_op(self, other, op=lambda a, b: b - a, zero=0)

    def __isub__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a - b, zero=0, result=self)

    def __mul__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a * b, zero=1)

    __rmul__ = __mul__

    def __imul__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a * b, zero=1, result=self)

    def __truediv__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a / b, zero=1)

    def __rtruediv__(self, other):
        return self.bin_op(self, other, op=lambda a, b: b / a, zero=1)

    def __floordiv__(self, other):
        return self.bin_op(self, other, op=lambda a, b: a // b, zero=1)

    def __neg__(self):
        return self.unary_op(op=lambda a: -a)

    def __bool__(self):
        return any(self.values())

    def elem_eq(self, other, result_with_default: bool = True) -> "NumbersDict":
        """element-wise equality"""

        def op(a, b):
            if a is None or b is None:
                return None
            return a == b

        res = self.bin_op(self, other, op=op, zero=None)
        if not result_with_default:
            res.value = None
        return res

    def __eq__(self, other):
        return all(v for v in self.elem_eq(other).values() if v is not None)

    def __ne__(self, other):
        return not (self == other)

    def __hash__(self):
        return id(self)

    def __cmp__(self, other):
        raise Exception("NumbersDict has no total order")

    def any_compare(self, other, cmp: Callable[[Any, Any], bool]) -> bool:
        """any(cmp(self[k], other[k]))"""
        for key in self.keys():
            if key in other.keys():
                if cmp(self[key], other[key]):
                    return True
            elif other.value is not None:
                if cmp(self[key], other.value):
                    return True
        if self.value is not None and other.value is not None:
            if cmp(self.value, other.value):
                return True
        return False

    @staticmethod
    def _max(*args):
        args = [a for a in args if a is not None]
        if not args:
            return None
        if len(args) == 1:
            return args[0]
        return builtins.max(*args)

    @staticmethod
    def _min(*args):
        args = [a for a in args if a is not None]
        if not args:
            return None
        if len(args) == 1:
            return args[0]
        return builtins.min(*args)

    @classmethod
    def max(cls, items) -> "NumbersDict":
        """element-wise max over items"""
        assert items
        if len(items) == 1:
            return NumbersDict(items[0])
        if len(items) == 2:
            return cls.bin_op(items[0], items[1], op=cls._max, zero=None)
        return cls.max([items[0], cls.max(items[1:])])

    @classmethod
    def min(cls, items) -> "NumbersDict":
        """element-wise min over items"""
        assert items
        if len(items) == 1:
            return NumbersDict(items[0])
        if len(items) == 2:
            return cls.bin_op(items[0], items[1], op=cls._min, zero=None)
        return cls.min([items[0], cls.min(items[1:])])

    @staticmethod
    def _max_error():
        raise Exception("Use max_value on an instance")

    def keys(self):
        """keys"""
        return self.dict.keys()

    def values(self):
        """values incl broadcast default"""
        return list(self.dict.values()) + ([self.value] if self.value is not None else [])

    def items(self):
        """items"""
        return self.dict.items()

    def has_value_for(self, key) -> bool:
        """key present or default"""
        return key in self.dict or self.value is not None

    def max_value(self):
        """max over values"""
        return builtins.max(self.values())

    def min_value(self):
        """min over values"""
        return builtins.min(self.values())

    def __repr__(self):
        if self.value is None and not self.dict:
            return "%s()" % self.__class__.__name__
        if self.value is None and self.dict:
            return "%s(%r)" % (self.__class__.__name__, self.dict)
        if not self.dict and self.value is not None:
            return "%s(%r)" % (self.__class__.__name__, self.value)
        return "%s(numbers_dict=%r, broadcast_value=%r)" % (self.__class__.__name__, self.dict, self.value)


class Stats:
    """
    Running mean / variance / min / max over arrays collected one sequence at a time (Welford-free: sums in float64).
    """

    def __init__(self, format_str=None):
        self.format_str = format_str or str
        self.mean = 0.0
        self.mean_sq = 0.0
        self.var = 0.0
        self.min = None
        self.max = None
        self.total_data_len = 0
        self.num_seqs = 0

    def collect(self, data):
        """:param numpy.ndarray data: shape (time, ...) or (time,)"""
        data = numpy.asarray(data)
        if data.ndim == 0:
            data = data.reshape(1)
        self.num_seqs += 1
        if data.shape[0] == 0:
            return
        new_total = self.total_data_len + data.shape[0]
        mean_diff = numpy.mean(data, axis=0) - self.mean
        m_a = self.var * self.total_data_len
        m_b = numpy.var(data, axis=0) * data.shape[0]
        m2 = m_a + m_b + mean_diff**2 * self.total_data_len * data.shape[0] / new_total
        self.var = m2 / new_total
        self.mean = self.mean + mean_diff * data.shape[0] / new_total
        self.total_data_len = new_total
        mn, mx = numpy.min(data, axis=0), numpy.max(data, axis=0)
        self.min = mn if self.min is None else numpy.minimum(self.min, mn)
        self.max = mx if self.max is None else numpy.maximum(self.max, mx)

    def get_mean(self):
        """mean"""
        return self.mean

    def get_std_dev(self):
        """std dev"""
        return numpy.sqrt(self.var)

    def dump(self, output_file_prefix=None, stream=None, stream_prefix=""):
        """print and/or write ``<prefix>.mean.txt`` / ``<prefix>.std_dev.txt``"""
        if stream is None:
            stream = sys.stdout
        print("%sStats:" % stream_prefix, file=stream)
        print("%s  %i seqs, %i total frames, %f average frames" % (
            stream_prefix, self.num_seqs, self.total_data_len, self.total_data_len / max(self.num_seqs, 1)), file=stream)
        print("%s  Mean: %s" % (stream_prefix, self.format_str(self.get_mean())), file=stream)
        print("%s  Std dev: %s" % (stream_prefix, self.format_str(self.get_std_dev())), file=stream)
        print("%s  Min/max: %s / %s" % (stream_prefix, self.format_str(self.min), self.format_str(self.max)), file=stream)
        if output_file_prefix:
            numpy.savetxt("%s.mean.txt" % output_file_prefix, numpy.atleast_1d(self.get_mean()))
            numpy.savetxt("%s.std_dev.txt" % output_file_prefix, numpy.atleast_1d(self.get_std_dev()))


def should_write_to_disk(config) -> bool:
    """
    Only the first rank of a distributed job writes models, LR file, logs of scores.

    :param returnn_b200.config.Config config:
    """
    if config is not None and config.typed_value("torch_distributed") is not None:
        from returnn_b200.torch import distributed as _dist

        ctx = _dist.get_ctx(config=config)
        if ctx is not None and ctx.rank() != 0:
            return False
    if config is not None and config.is_true("dry_run"):
        return False
    return True


def slurm_time_left_sec() -> Optional[float]:
    """seconds left of the surrounding SLURM job, None if not under SLURM or unknown"""
    job_id = os.environ.get("SLURM_JOB_ID")
    if not job_id:
        return None
    import subprocess

    try:
        out = subprocess.check_output(["squeue", "-h", "-j", job_id, "-O", "TimeLeft"], timeout=10).decode().strip()
    except Exception:
        return None
    # [days-]hours:minutes:seconds
    m = re.match(r"^(?:(\d+)-)?(?:(\d+):)?(\d+):(\d+)$", out)
    if not m:
        return None
    d, h, mi, s = (int(x) if x else 0 for x in m.groups())
    return float(((d * 24 + h) * 60 + mi) * 60 + s)


class LockFile:
    """Directory-scoped lock file with stale-lock detection (pid + mtime)."""

    def __init__(self, directory: str, name: str = "lock_file", lock_timeout: float = 60 * 60):
        self.directory = directory
        self.name = name
        self.fd = None
        self.lock_timeout = lock_timeout
        self.lockfile = "%s/%s" % (directory, name)

    def is_old_lockfile(self) -> bool:
        """stale by mtime or dead owner"""
        try:
            mtime = os.path.getmtime(self.lockfile)
        except OSError:
            return False
        if time.time() - mtime > self.lock_timeout:
            return True
        try:
            pid = int(open(self.lockfile).read().strip() or -1)
        except (OSError, ValueError):
            return False
        if pid > 0:
            try:
                os.kill(pid, 0)
            except ProcessLookupError:
                return True
            except OSError:
                return False
        return False

    def maybe_remove_old_lockfile(self):
        """remove stale"""
        if self.is_old_lockfile():
            try:
                os.remove(self.lockfile)
            except OSError:
                pass

    def is_locked(self) -> bool:
        """held by someone"""
        self.maybe_remove_old_lockfile()
        return os.path.exists(self.lockfile)

    def lock(self):
        """block until acquired"""
        os.makedirs(self.directory, exist_ok=True)
        while True:
            try:
                self.fd = os.open(self.lockfile, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
                os.write(self.fd, ("%i\n" % os.getpid()).encode())
                return
            except FileExistsError:
                self.maybe_remove_old_lockfile()
                time.sleep(0.05)

    def unlock(self):
        """release"""
        if self.fd is not None:
            os.close(self.fd)
            self.fd = None
        try:
            os.remove(self.lockfile)
        except OSError:
            pass

    def __enter__(self):
        self.lock()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.unlock()


def compute_bleu(reference_corpus, translation_corpus, max_order: int = 4, use_bp: bool = True) -> float:
    """
    Corpus BLEU over token lists.

    :param list[list[str]] reference_corpus:
    :param list[list[str]] translation_corpus:
    """
    reference_length = 0
    translation_length = 0
    matches_by_order = [0] * max_order
    possible_matches_by_order = [0] * max_order

    def ngrams(seg):
        c = collections.Counter()
        for order in range(1, max_order + 1):
            for i in range(0, len(seg) - order + 1):
                c[tuple(seg[i : i + order])] += 1
        return c

    for ref, hyp in zip(reference_corpus, translation_corpus):
        reference_length += len(ref)
        translation_length += len(hyp)
        ref_c, hyp_c = ngrams(ref), ngrams(hyp)
        overlap = {ng: builtins.min(cnt, hyp_c[ng]) for ng, cnt in ref_c.items()}
        for ng, cnt in overlap.items():
            matches_by_order[len(ng) - 1] += cnt
        for ng, cnt in hyp_c.items():
            possible_matches_by_order[len(ng) - 1] += cnt
    precisions = [0.0] * max_order
    smooth = 1.0
    for i in range(max_order):
        if possible_matches_by_order[i] > 0:
            if matches_by_order[i] > 0:
                precisions[i] = matches_by_order[i] / possible_matches_by_order[i]
            else:
                smooth *= 2
                precisions[i] = 1.0 / (smooth * possible_matches_by_order[i])
    geo_mean = math.exp(sum(math.log(p) for p in precisions if p) / max_order) if builtins.max(precisions) > 0 else 0.0
    bp = 1.0
    if use_bp and translation_length:
        ratio = translation_length / builtins.max(reference_length, 1)
        bp = math.exp(1 - 1.0 / ratio) if ratio < 1.0 else 1.0
    return float(geo_mean * bp)


def try_run(func, args=(), catch_exc=Exception, default=None):
    """call, swallow exceptions"""
    try:
        return func(*args)
    except catch_exc:
        return default


def class_idx_seq_to_1_of_k(seq, num_classes: int):
    """int seq -> one-hot float32 matrix"""
    seq = numpy.asarray(seq)
    out = numpy.zeros((len(seq), num_classes), dtype="float32")
    out[numpy.arange(len(seq)), seq] = 1.0
    return out


def binary_search_any(cmp: Callable[[int], int], low: int, high: int) -> Optional[int]:
    """find any i in [low, high) with cmp(i) == 0; cmp gives -1 if i too low, 1 if too high"""
    while low < high:
        mid = (low + high) // 2
        r = cmp(mid)
        if r < 0:
            low = mid + 1
        elif r > 0:
            high = mid
        else:
            return mid
    return None


def to_bool(v) -> bool:
    """string/number -> bool with the usual spellings"""
    try:
        return bool(int(v))
    except (ValueError, TypeError):
        pass
    if isinstance(v, str):
        v = v.lower()
        if v in ("true", "yes", "on", "1"):
            return True
        if v in ("false", "no", "off", "0"):
            return False
    raise ValueError("to_bool cannot handle %r" % (v,))


def as_str(s) -> str:
    """bytes/str -> str"""
    if isinstance(s, str):
        return s
    if isinstance(s, bytes):
        return s.decode("utf8")
    return str(s)


def is_running_on_cluster() -> bool:
    """SGE/SLURM environment"""
    return bool(os.environ.get("SLURM_JOB_ID") or os.environ.get("JOB_ID"))


def read_pickled_object(p, encoding=None):
    """
    One object written by ``write_pickled_object``: an int32 length, then that many bytes of pickle.
    Raises EOFError when the stream ends first. Parity: returnn/util/basic.py ``read_pickled_object``.
    """
    import pickle
    import struct

    def exactly(n):
        parts = []
        while n > 0:
            b = p.read(n)
            if not b:
                raise EOFError("stream ended inside a pickled object")
            parts.append(b)
            n -= len(b)
        return b"".join(parts)

    (size,) = struct.unpack("<i", exactly(4))
    assert size > 0, "read_pickled_object: size %i" % size
    data = exactly(size)
    return pickle.loads(data) if encoding is None else pickle.loads(data, encoding=encoding)


def better_repr(o) -> str:
    """deterministic repr for dicts (sorted keys), used by config diff"""
    if isinstance(o, dict):
        return "{\n%s}" % "".join("%s: %s,\n" % (better_repr(k), better_repr(v)) for k, v in sorted(o.items(), key=lambda kv: str(kv[0])))
    if isinstance(o, (list, tuple)):
        inner = ", ".join(better_repr(v) for v in o)
        if isinstance(o, list):
            return "[%s]" % inner
        return "(%s%s)" % (inner, "," if len(o) == 1 else "")
    return repr(o)


@contextlib.contextmanager
def override_env_var(var_name: str, value: str):
    """temporarily set env var"""
    old = os.environ.get(var_name)
    os.environ[var_name] = value
    try:
        yield
    finally:
        if old is None:
            os.environ.pop(var_name, None)
        else:
            os.environ[var_name] = old


def get_temp_dir(with_username: bool = True) -> str:
    """scratch dir"""
    base = os.environ.get("TMPDIR", "/tmp")
    if with_username:
        base = os.path.join(base, get_login_username())
    os.makedirs(base, exist_ok=True)
    return base


def get_cache_dir() -> str:
    """cache dir for compiled native code"""
    d = os.environ.get("RETURNN_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "returnn_b200")
    os.makedirs(d, exist_ok=True)
    return d


def deep_update_dict_values(d: Dict, key, new_value):
    """set key everywhere in nested dict"""
    for v in d.values():
        if isinstance(v, dict):
            deep_update_dict_values(v, key=key, new_value=new_value)
    if key in d:
        d[key] = new_value


def next_power_of_two(n: int) -> int:
    """smallest power of two >= n"""
    return 1 << (int(n) - 1).bit_length() if n > 1 else 1


def ceil_div(a: int, b: int) -> int:
    """-(-a // b)"""
    return -(-a // b)


def cf(filename: str) -> str:
    """cached file path via the file cache when configured, else identity"""
    from .file_cache import get_instance_if_enabled

    fc = get_instance_if_enabled()
    if fc is None:
        return filename
    return fc.get_file(filename)


from .basic_more import *  # noqa: E402,F401,F403  (the smaller helpers of this module live in basic_more.py)
from .basic_more import _eq as _eq_generic  # noqa: E402,F401
