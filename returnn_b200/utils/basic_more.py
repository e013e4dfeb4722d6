"""
The small general-purpose helpers of the utility module that configs, tools and user code of the reference use by name: shell and git
queries, checkpoint file names, terminal helpers, pretty printing, dict / object helpers, threads, array helpers, orthography parsing,
introspection of constructors, hashing helpers, file and environment helpers, machine queries. All of them are re-exported from
:mod:`returnn_b200.utils.basic`. Parity: returnn/util/basic.py (same names, own implementations).
"""

from __future__ import annotations
import contextlib
import functools
import inspect
import json
import os
import re
import shutil
import subprocess
import sys
import threading
import time
import types
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Type, TypeVar, Union
import numpy

T = TypeVar("T")


# ---- platform, versions, shell ------------------------------------------------------------------------------------------------
def is_64bit_platform() -> bool:
    """pointer size of this interpreter"""
    return sys.maxsize > 2 ** 32


def sys_cmd_out_lines(cmd: str) -> List[str]:
    """stdout lines of a shell command; raises on a non-zero exit code"""
    res = subprocess.run(cmd, shell=True, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, check=True)
    return res.stdout.splitlines()


def sys_exec_out(*args: str, **kwargs) -> str:
    """stdout of ``args`` (no shell); raises ``CalledProcessError`` on failure"""
    return subprocess.run(list(args), stdout=subprocess.PIPE, text=True, check=True, **kwargs).stdout


def sys_exec_ret_code(*args: str, **kwargs) -> int:
    """exit code of ``args`` (no shell), output discarded"""
    return subprocess.run(list(args), stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, **kwargs).returncode


def _git(git_dir: str, *args: str) -> str:
    return sys_exec_out("git", *args, cwd=git_dir, stderr=subprocess.DEVNULL).strip()


def git_commit_rev(commit: str = "HEAD", git_dir: str = ".", length: Optional[int] = 10) -> str:
    """abbreviated hash of a commit"""
    rev = _git(git_dir, "rev-parse", commit)
    return rev[:length] if length else rev


def git_is_dirty(git_dir: str = ".") -> bool:
    """uncommitted changes in the work tree"""
    return sys_exec_ret_code("git", "diff", "--quiet", "HEAD", cwd=git_dir) != 0


def git_commit_date(commit: str = "HEAD", git_dir: str = ".") -> str:
    """commit time as ``YYYYMMDD.HHMMSS`` (UTC)"""
    ts = int(_git(git_dir, "show", "-s", "--format=%ct", commit))
    return time.strftime("%Y%m%d.%H%M%S", time.gmtime(ts))


def git_describe_head_version(git_dir: str = ".") -> str:
    """``<commit date>--git-<hash>[-dirty]``"""
    return "%s--git-%s%s" % (git_commit_date(git_dir=git_dir), git_commit_rev(git_dir=git_dir), "-dirty" if git_is_dirty(git_dir) else "")


def describe_returnn_version() -> str:
    """version string of this package: from git when it is a checkout, else the package version"""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        return git_describe_head_version(git_dir=here)
    except Exception:
        try:
            from .. import __version__

            return str(__version__)
        except Exception:
            return "unknown"


def describe_torch_version() -> str:
    """torch version and where it was loaded from"""
    import torch

    return "%s (%s in %s)" % (torch.__version__, getattr(torch.version, "git_version", "?")[:10], os.path.dirname(torch.__file__))


def describe_tensorflow_version() -> str:
    """there is no TensorFlow backend in this framework"""
    return "<not used>"


def get_tensorflow_version_tuple() -> Tuple[int, ...]:
    """there is no TensorFlow backend in this framework"""
    return ()


def eval_shell_env(token: str) -> str:
    """``$VAR`` -> value of the environment variable (empty if unset), anything else unchanged"""
    if token.startswith("$"):
        return os.environ.get(token[1:], "")
    return token


def eval_shell_str(s: Union[str, Callable[[], Union[str, Sequence[str]]], Sequence[str]]) -> List[str]:
    """a command line as string (shell quoting rules, ``$VAR`` tokens expanded), list, or function returning either -> argv list"""
    import shlex

    if callable(s):
        s = s()
    tokens = shlex.split(s) if isinstance(s, str) else list(s)
    return [eval_shell_env(t) for t in tokens]


def expand_env_vars(s: str) -> str:
    """``$VAR`` and ``${VAR}`` inside a string"""
    return os.path.expandvars(s)


def which(program: str) -> Optional[str]:
    """full path of an executable on PATH or None"""
    return shutil.which(program)


def which_pip() -> List[str]:
    """argv prefix that runs pip for this interpreter"""
    return [sys.executable, "-m", "pip"]


def pip_check_is_installed(package: str) -> bool:
    """whether a distribution of this name is installed"""
    try:
        from importlib import metadata

        metadata.version(package)
        return True
    except Exception:
        return False


def pip_install(*pkg_names: str):
    """``pip install`` for this interpreter (needs an index or a wheelhouse configured in pip's environment)"""
    subprocess.run(which_pip() + ["install"] + list(pkg_names), check=True)


# ---- checkpoint file names ---------------------------------------------------------------------------------------------------------
def get_model_filename_postfix() -> str:
    """extension of a parameter checkpoint"""
    return ".pt"


def get_checkpoint_filepattern(filepath: str) -> str:
    """``<model>.<epoch>.pt`` -> ``<model>.<epoch>`` (what ``load`` / ``import_model_train_epoch1`` take)"""
    for ext in (".opt.pt", ".pt", ".meta", ".index"):
        if filepath.endswith(ext):
            return filepath[: -len(ext)]
    return filepath


def model_epoch_from_filename(filename: str) -> int:
    """epoch number out of ``<model>.<epoch>[.pt]`` (a ``.pretrain`` infix is allowed)"""
    m = re.match(r".*\.(?:pretrain\.)?([0-9]+)(?:\.opt)?(?:\.pt|\.meta|\.index)?$", filename)
    assert m, "no epoch in model filename %r" % filename
    return int(m.group(1))


# ---- terminal ----------------------------------------------------------------------------------------------------------------------
def terminal_size(file=sys.stdout) -> Tuple[int, int]:
    """(columns, rows), (-1, -1) if not a terminal"""
    try:
        sz = os.get_terminal_size(file.fileno())
        return sz.columns, sz.lines
    except Exception:
        return -1, -1


def is_tty(file=sys.stdout) -> bool:
    """whether the stream is a terminal"""
    try:
        return bool(file.isatty())
    except Exception:
        return False


def confirm(txt: str, exit_on_false: bool = False) -> bool:
    """ask ``txt (y/n)`` on the terminal"""
    while True:
        ans = input("%s Confirm? [yes/no] " % txt).strip().lower()
        if ans in ("y", "yes"):
            return True
        if ans in ("n", "no"):
            if exit_on_false:
                sys.exit(1)
            return False
        print("Please answer yes or no.")


_pp_limit = 300
_pp_as_bytes = False


def set_pretty_print_default_limit(limit: Optional[int]):
    """collections longer than this are abbreviated by :func:`pretty_print` (None: never)"""
    global _pp_limit
    _pp_limit = limit


def set_pretty_print_as_bytes(as_bytes: bool):
    """whether strings are printed as bytes literals"""
    global _pp_as_bytes
    _pp_as_bytes = as_bytes


def pretty_print(obj: Any, limit: Optional[int] = None) -> str:
    """``repr`` with one item per line for nested containers; the result is valid Python as long as nothing is cut"""
    from .pprint import pformat

    limit = _pp_limit if limit is None else limit
    if limit is not None and isinstance(obj, (list, tuple, dict, set)) and len(obj) > limit:
        if isinstance(obj, dict):
            obj = dict(list(obj.items())[:limit])
        else:
            obj = type(obj)(list(obj)[:limit])
        return pformat(obj) + "  # ... cut at %i items" % limit
    s = pformat(obj)
    return repr(s.encode("utf8")) if _pp_as_bytes and isinstance(obj, str) else s


def progress_bar(complete: float = 1.0, prefix: str = "", suffix: str = "", file=None):
    """one-line text progress bar on a terminal (no output elsewhere); ``complete`` in [0, 1]"""
    file = file or sys.stdout
    cols, _ = terminal_size(file)
    if cols <= 0:
        return
    if complete >= 1.0:
        file.write("\r%s\r" % (" " * (cols - 1)))
        file.flush()
        return
    width = max(cols - len(prefix) - len(suffix) - 12, 5)
    n = int(max(min(complete, 1.0), 0.0) * width)
    file.write("\r%s[%s%s] %5.1f%% %s" % (prefix + " " if prefix else "", "=" * n, " " * (width - n), complete * 100.0, suffix))
    file.flush()


_pb_start: Dict[str, float] = {}


def progress_bar_with_time(complete: float = 1.0, prefix: str = "", **kwargs):
    """:func:`progress_bar` with the estimated remaining time as suffix"""
    from .basic import hms

    key = prefix
    now = time.time()
    if key not in _pb_start or complete <= 0:
        _pb_start[key] = now
    suffix = ""
    if complete > 0:
        elapsed = now - _pb_start[key]
        suffix = "%s remaining" % hms(elapsed / complete * (1.0 - complete))
    if complete >= 1.0:
        _pb_start.pop(key, None)
    progress_bar(complete, prefix=prefix, suffix=suffix, **kwargs)


# ---- memory, machine ---------------------------------------------------------------------------------------------------------------
def available_physical_memory_in_bytes() -> int:
    """free + reclaimable RAM"""
    try:
        import psutil

        return int(psutil.virtual_memory().available)
    except Exception:
        return int(os.sysconf("SC_AVPHYS_PAGES") * os.sysconf("SC_PAGE_SIZE"))


def default_cache_size_in_gbytes(factor: float = 0.7) -> int:
    """a share of the available memory, for dataset caches"""
    return int(available_physical_memory_in_bytes() * factor / (1024 ** 3))


def read_sge_num_procs(job_id: Optional[str] = None) -> Optional[int]:
    """slots of the current Grid Engine job (``NSLOTS``) or None"""
    v = os.environ.get("NSLOTS")
    return int(v) if v and v.isdigit() else None


def get_number_available_cpus() -> int:
    """CPUs this process may run on"""
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def guess_requested_max_num_threads(log_file=None, fallback_num_cpus: bool = True) -> Optional[int]:
    """what the batch system or the environment asked for: SGE slots, Slurm CPUs per task, ``OMP_NUM_THREADS``; else the CPU count"""
    for name in ("NSLOTS", "SLURM_CPUS_PER_TASK", "OMP_NUM_THREADS"):
        v = os.environ.get(name)
        if v and v.isdigit():
            if log_file:
                print("%s is set to %s." % (name, v), file=log_file)
            return int(v)
    return get_number_available_cpus() if fallback_num_cpus else None


def get_cpu_model_name() -> str:
    """as ``/proc/cpuinfo`` has it"""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    import platform

    return platform.processor() or "unknown"


def get_gpu_names() -> List[str]:
    """names of the visible CUDA devices"""
    try:
        import torch

        return [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
    except Exception:
        return []


def get_num_gpu_devices() -> Tuple[Optional[int], int]:
    """(cores per device: unknown, number of devices)"""
    return None, len(get_gpu_names())


def have_gpu() -> bool:
    """a CUDA device is visible"""
    return get_num_gpu_devices()[1] > 0


def get_lsb_release() -> Dict[str, str]:
    """``/etc/lsb-release`` (or ``os-release``) as a dict"""
    out: Dict[str, str] = {}
    for fn in ("/etc/lsb-release", "/etc/os-release"):
        if os.path.exists(fn):
            with open(fn) as f:
                for line in f:
                    k, sep, v = line.strip().partition("=")
                    if sep:
                        out[k] = v.strip('"')
            break
    return out


def get_ubuntu_major_version() -> Optional[int]:
    """e.g. 22, None on other systems"""
    d = get_lsb_release()
    if d.get("DISTRIB_ID", d.get("ID", "")).lower() != "ubuntu":
        return None
    v = d.get("DISTRIB_RELEASE", d.get("VERSION_ID", ""))
    return int(float(v)) if v else None


def parse_ld_conf_file(fn: str) -> List[str]:
    """library directories named by an ``ld.so.conf`` file (``include`` lines followed)"""
    import glob as _glob

    paths: List[str] = []
    try:
        with open(fn) as f:
            for line in f:
                line = line.split("#", 1)[0].strip()
                if not line:
                    continue
                if line.startswith("include "):
                    for sub in _glob.glob(line[len("include "):].strip()):
                        paths.extend(parse_ld_conf_file(sub))
                else:
                    paths.append(line)
    except OSError:
        pass
    return paths


def get_ld_paths() -> List[str]:
    """where the dynamic linker looks: ``LD_LIBRARY_PATH``, ``/etc/ld.so.conf``, the defaults"""
    paths = [p for p in os.environ.get("LD_LIBRARY_PATH", "").split(":") if p]
    paths += parse_ld_conf_file("/etc/ld.so.conf")
    paths += ["/lib", "/usr/lib", "/lib64", "/usr/lib64"]
    seen, out = set(), []
    for p in paths:
        if p not in seen:
            seen.add(p)
            out.append(p)
    return out


def find_lib(lib_name: str) -> Optional[str]:
    """first file of that name on the linker's search path"""
    for p in get_ld_paths():
        fn = os.path.join(p, lib_name)
        if os.path.exists(fn):
            return fn
    return None


def make_dll_name(basename: str) -> str:
    """``lib<name>.so`` (``.dylib`` on macOS)"""
    return "lib%s.%s" % (basename, "dylib" if sys.platform == "darwin" else "so")


def escape_c_str(s: str) -> str:
    """a C string literal (with the quotes) for arbitrary text"""
    out = []
    for ch in s.encode("utf8"):
        c = chr(ch)
        if c in '\\"':
            out.append("\\" + c)
        elif c == "\n":
            out.append("\\n")
        elif 32 <= ch < 127:
            out.append(c)
        else:
            out.append('\\%03o' % ch)
    return '"%s"' % "".join(out)


# ---- dicts, objects -----------------------------------------------------------------------------------------------------------------
class ObjAsDict:
    """the attributes of an object through the mapping interface"""

    def __init__(self, obj: Any):
        self.__obj = obj

    def __getitem__(self, item):
        if not isinstance(item, str):
            raise KeyError(item)
        try:
            return getattr(self.__obj, item)
        except AttributeError as e:
            raise KeyError(e)

    def __contains__(self, item):
        return isinstance(item, str) and hasattr(self.__obj, item)

    def items(self):
        """like dict.items over the instance dict"""
        return vars(self.__obj).items()


class DictAsObj:
    """the keys of a dict as attributes"""

    def __init__(self, dikt: Dict[str, Any]):
        self.__dict__ = dikt


def dict_joined(*ds: Dict[Any, Any]) -> Dict[Any, Any]:
    """later dicts win"""
    res: Dict[Any, Any] = {}
    for d in ds:
        res.update(d)
    return res


def dict_zip(keys: Sequence[Any], values: Sequence[Any]) -> Dict[Any, Any]:
    """``dict(zip(...))`` with a check of the lengths"""
    assert len(keys) == len(values), "dict_zip: %i keys, %i values" % (len(keys), len(values))
    return dict(zip(keys, values))


def sorted_values_from_dict(d: Dict[Any, Any]) -> List[Any]:
    """values in the order of the sorted keys"""
    return [v for _, v in sorted(d.items())]


def obj_diff_list(self: Any, other: Any, **kwargs) -> List[str]:
    """human-readable differences of two nested structures (dicts, lists, tuples, sets, leaves by ``==``), empty when equal"""
    prefix = kwargs.get("_prefix", "")
    allowed = kwargs.get("allowed_mapping")
    if self is None and other is None:
        return []
    if type(self) is not type(other) and not (isinstance(self, (int, float)) and isinstance(other, (int, float))):
        return ["%stype diff: self is %s but other is %s" % (prefix, type(self).__name__, type(other).__name__)]
    if isinstance(self, dict):
        out = []
        for k in sorted(set(self) | set(other), key=repr):
            if k not in self:
                out.append("%skey %r not in self" % (prefix, k))
            elif k not in other:
                out.append("%skey %r not in other" % (prefix, k))
            else:
                out += obj_diff_list(self[k], other[k], _prefix="%s[%r] " % (prefix.rstrip(), k), allowed_mapping=allowed)
        return out
    if isinstance(self, (list, tuple)):
        if len(self) != len(other):
            return ["%slist diff len: len self: %i, len other: %i" % (prefix, len(self), len(other))]
        out = []
        for i, (a, b) in enumerate(zip(self, other)):
            out += obj_diff_list(a, b, _prefix="%s[%i] " % (prefix.rstrip(), i), allowed_mapping=allowed)
        return out
    if isinstance(self, set):
        out = ["%sitem %r not in other" % (prefix, x) for x in sorted(self - other, key=repr)]
        out += ["%sitem %r not in self" % (prefix, x) for x in sorted(other - self, key=repr)]
        return out
    if self != other and not (allowed and allowed(self, other)):
        return ["%sself: %r != other: %r" % (prefix, self, other)]
    return []


def obj_diff_str(self: Any, other: Any, **kwargs) -> str:
    """:func:`obj_diff_list` joined by newlines, or "No diff." """
    diff = obj_diff_list(self, other, **kwargs)
    return "\n".join(diff) if diff else "No diff."


def find_ranges(ls: Sequence[int]) -> List[Tuple[int, int]]:
    """sorted integers -> maximal ``(start, end)`` ranges, end exclusive: [1, 2, 3, 7, 8] -> [(1, 4), (7, 9)]"""
    out: List[Tuple[int, int]] = []
    for v in ls:
        if out and out[-1][1] == v:
            out[-1] = (out[-1][0], v + 1)
        else:
            out.append((v, v + 1))
    return out


def uniq_generic(ls: Iterable[T]) -> List[T]:
    """first occurrences in order, for items that need not be hashable"""
    out: List[T] = []
    for x in ls:
        if not any(x is y or _eq(x, y) for y in out):
            out.append(x)
    return out


def _eq(a, b) -> bool:
    try:
        r = a == b
        return bool(r.all()) if hasattr(r, "all") else bool(r)
    except Exception:
        return False


class FrozenDict(dict):
    """hashable, immutable dict"""

    def _blocked(self, *a, **kw):
        raise TypeError("FrozenDict is immutable")

    __setitem__ = __delitem__ = clear = pop = popitem = setdefault = update = _blocked  # type: ignore[assignment]

    def __hash__(self):  # type: ignore[override]
        return hash(frozenset((k, make_hashable(v)) for k, v in self.items()))


def make_hashable(obj: Any) -> Any:
    """nested lists / dicts / sets / arrays as tuples / frozen dicts / frozen sets, so that the result can be a dict key"""
    if isinstance(obj, dict):
        return FrozenDict((make_hashable(k), make_hashable(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return tuple(make_hashable(x) for x in obj)
    if isinstance(obj, (set, frozenset)):
        return frozenset(make_hashable(x) for x in obj)
    if isinstance(obj, numpy.ndarray):
        return (obj.shape, obj.dtype.str, obj.tobytes())
    hash(obj)
    return obj


class RefIdEq:
    """wraps an object so that equality and hash are identity"""

    def __init__(self, obj: Any):
        self.obj = obj

    def __hash__(self):
        return id(self.obj)

    def __eq__(self, other):
        return isinstance(other, RefIdEq) and self.obj is other.obj

    def __ne__(self, other):
        return not self == other


class DictRefKeys:
    """dict keyed by object identity (keys need not be hashable; they are kept alive)"""

    def __init__(self):
        self._d: Dict[RefIdEq, Any] = {}

    def __setitem__(self, key, value):
        self._d[RefIdEq(key)] = value

    def __getitem__(self, key):
        return self._d[RefIdEq(key)]

    def __delitem__(self, key):
        del self._d[RefIdEq(key)]

    def __contains__(self, key):
        return RefIdEq(key) in self._d

    def __len__(self):
        return len(self._d)

    def __iter__(self):
        return (k.obj for k in self._d)

    def get(self, key, default=None):
        """as dict.get"""
        return self._d.get(RefIdEq(key), default)

    def items(self):
        """(key object, value) pairs"""
        return [(k.obj, v) for k, v in self._d.items()]


def attr_chain(base: Any, attribs: Union[str, Sequence[str]]) -> Any:
    """``base.a.b.c`` for ``attribs = ["a", "b", "c"]`` (or the single name)"""
    if isinstance(attribs, str):
        attribs = [attribs]
    for a in attribs:
        base = getattr(base, a)
    return base


def is_namedtuple(cls: Any) -> bool:
    """a class made by ``collections.namedtuple`` / ``typing.NamedTuple``"""
    return isinstance(cls, type) and issubclass(cls, tuple) and hasattr(cls, "_fields") and hasattr(cls, "_make")


def ensure_list_of_type(ls: Any, type_: Type[T]) -> List[T]:
    """list (or tuple) whose items all are of the type -> list; anything else raises"""
    assert isinstance(ls, (list, tuple)), "expected a list, got %r" % type(ls)
    for x in ls:
        assert isinstance(x, type_), "expected items of %s, got %r" % (type_.__name__, type(x))
    return list(ls)


def camel_case_to_snake_case(name: str) -> str:
    """``HelloWorldHTTP`` -> ``hello_world_http``"""
    s = re.sub(r"(.)([A-Z][a-z]+)", r"\1_\2", name)
    return re.sub(r"([a-z0-9])([A-Z])", r"\1_\2", s).lower()


def str_is_number(s: str) -> bool:
    """parses as float"""
    try:
        float(s)
        return True
    except (TypeError, ValueError):
        return False


def unicode_to_str(s: Any) -> str:
    """bytes are decoded as utf8, everything else goes through ``str``"""
    return s.decode("utf8") if isinstance(s, bytes) else str(s)


def deepcopy(x: T, stop_types: Optional[Sequence[type]] = None) -> T:
    """``copy.deepcopy`` that passes instances of ``stop_types`` through by reference"""
    import copy

    memo: Dict[int, Any] = {}
    if stop_types:
        stop = tuple(stop_types)

        def walk(o):
            if isinstance(o, stop):
                memo[id(o)] = o
            elif isinstance(o, dict):
                for v in o.values():
                    walk(v)
            elif isinstance(o, (list, tuple, set)):
                for v in o:
                    walk(v)
            elif hasattr(o, "__dict__"):
                for v in vars(o).values():
                    walk(v)

        walk(x)
    return copy.deepcopy(x, memo)


# ---- threads -----------------------------------------------------------------------------------------------------------------------
_quitting = False


def start_daemon_thread(target: Callable, args: Sequence[Any] = ()) -> threading.Thread:
    """start and return a daemon thread"""
    t = threading.Thread(target=target, args=tuple(args), daemon=True)
    t.start()
    return t


def is_quitting() -> bool:
    """the interpreter is shutting down (or :func:`interrupt_main` was called)"""
    return _quitting or sys.is_finalizing()


def interrupt_main():
    """KeyboardInterrupt in the main thread, from any thread"""
    global _quitting
    _quitting = True
    import _thread

    _thread.interrupt_main()


def init_thread_join_hack():
    """kept for configs that call it: joins are interruptible in Python 3 without any patch"""


class AsyncThreadRun(threading.Thread):
    """runs ``func`` in a daemon thread; :meth:`get` joins and returns its result (or re-raises its exception)"""

    def __init__(self, name: str, func: Callable[[], T]):
        super().__init__(name=name, daemon=True)
        self.func = func
        self.result: Any = None
        self.exc: Optional[BaseException] = None
        self.start()

    def run(self):
        try:
            self.result = self.func()
        except BaseException as e:
            self.exc = e

    def get(self) -> Any:
        """result of ``func``"""
        self.join()
        if self.exc is not None:
            raise self.exc
        return self.result


def wrap_async_func(f: Callable[[], T]) -> T:
    """run ``f`` in another thread and wait for it (so that the main thread stays responsive to signals)"""
    return AsyncThreadRun("wrap_async_func", f).get()


def try_and_ignore_exception(f: Callable[[], Any]):
    """call ``f``; an exception is printed, not raised"""
    try:
        f()
    except Exception as exc:
        print("Ignoring exception %s: %s" % (type(exc).__name__, exc), file=sys.stderr)


def try_get_stack_frame(depth: int = 1):
    """frame ``depth`` levels above the caller, or None"""
    try:
        return sys._getframe(depth + 1)
    except ValueError:
        return None


def try_get_caller_name(depth: int = 1, fallback: Optional[str] = None) -> Optional[str]:
    """function name ``depth`` levels above the caller"""
    f = try_get_stack_frame(depth + 1)
    return f.f_code.co_name if f is not None else fallback


def traceback_clear_frames(tb):
    """drop the local variables kept alive by a traceback"""
    while tb is not None:
        try:
            tb.tb_frame.clear()
        except RuntimeError:
            pass  # still running
        tb = tb.tb_next


class InfiniteRecursionDetected(Exception):
    """raised by :func:`guard_infinite_recursion`"""


_recursion_guard = threading.local()


@contextlib.contextmanager
def guard_infinite_recursion(*args):
    """``with guard_infinite_recursion(func, arg...):`` raises if the same key is entered again inside the block (same thread)"""
    active = getattr(_recursion_guard, "active", None)
    if active is None:
        active = _recursion_guard.active = set()
    key = tuple(id(a) if not isinstance(a, (str, int, float, tuple)) else a for a in args)
    if key in active:
        raise InfiniteRecursionDetected("infinite recursion detected: %r" % (args,))
    active.add(key)
    try:
        yield
    finally:
        active.discard(key)


# ---- arrays ------------------------------------------------------------------------------------------------------------------------
def prod(ls: Iterable[Any]) -> Any:
    """product of the items (1 for none)"""
    return functools.reduce(lambda a, b: a * b, ls, 1)


def slice_pad_zeros(x: numpy.ndarray, begin: int, end: int, axis: int = 0) -> numpy.ndarray:
    """``x[begin:end]`` along ``axis`` where the range may reach outside of the array: the missing part is zeros"""
    assert axis == 0, "slice_pad_zeros: only the first axis"
    pad_left = max(-begin, 0)
    pad_right = max(end - x.shape[0], 0)
    core = x[max(begin, 0): max(min(end, x.shape[0]), 0)]
    widths = [(pad_left, pad_right)] + [(0, 0)] * (x.ndim - 1)
    out = numpy.pad(core, widths)
    assert out.shape[0] == max(end - begin, 0) or end <= begin
    return out


def random_orthogonal(shape: Sequence[int], gain: float = 1.0, seed: Optional[int] = None) -> numpy.ndarray:
    """random matrix with orthonormal rows or columns (from the SVD of a Gaussian matrix), reshaped to ``shape``"""
    rng = numpy.random.RandomState(seed)
    flat = (shape[0], int(numpy.prod(shape[1:])))
    a = rng.normal(0.0, 1.0, flat)
    u, _, v = numpy.linalg.svd(a, full_matrices=False)
    q = u if u.shape == flat else v
    return (gain * q.reshape(shape)).astype("float32")


def inplace_increment(x: numpy.ndarray, idx: numpy.ndarray, y: numpy.ndarray) -> numpy.ndarray:
    """``x[idx] += y`` where repeated indices all count"""
    numpy.add.at(x, idx, y)
    return x


def softmax(x: numpy.ndarray, axis: Optional[int] = None) -> numpy.ndarray:
    """numerically stable softmax in numpy"""
    e = numpy.exp(x - numpy.max(x, axis=axis, keepdims=True))
    return e / numpy.sum(e, axis=axis, keepdims=True)


def validate_broadcast_all_sources(allow_broadcast_all_sources, inputs, common) -> None:
    """an op that broadcasts ALL of its inputs to a new shape must have been told that this is intended"""
    if allow_broadcast_all_sources is True or allow_broadcast_all_sources is None:
        return
    raise ValueError("all inputs %r are broadcast to %r: set allow_broadcast_all_sources=True if that is intended" % (inputs, common))


def load_txt_vector(filename: str) -> List[float]:
    """one number per line"""
    with open(filename) as f:
        return [float(line) for line in f if line.strip()]


def get_global_inf_value() -> float:
    """the value used for "minus infinity" in masks (config ``inf_value``, default ``inf``)"""
    try:
        from ..config import get_global_config

        cfg = get_global_config(raise_exception=False)
        if cfg is not None:
            return float(cfg.float("inf_value", float("inf")))
    except Exception:
        pass
    return float("inf")


def is_onnx_export_global() -> bool:
    """config ``onnx_export``: models then avoid ops the exporter cannot express"""
    try:
        from ..config import get_global_config

        cfg = get_global_config(raise_exception=False)
        return bool(cfg.bool("onnx_export", False)) if cfg is not None else False
    except Exception:
        return False


# ---- orthography ---------------------------------------------------------------------------------------------------------------------
def parse_orthography_into_symbols(orthography: str, upper_case_special: bool = True, word_based: bool = False, square_brackets_for_specials: bool = True) -> List[str]:
    """
    Characters (or words) of a transcription; ``[NOISE]``-style tokens stay one symbol.
    ``"hi [LAUGH] you"`` -> ``["h", "i", " ", "[LAUGH]", " ", "y", "o", "u"]``
    """
    out: List[str] = []
    parts = re.split(r"(\[[^\]]*\])", orthography.strip()) if square_brackets_for_specials else [orthography.strip()]
    for part in parts:
        if not part:
            continue
        if square_brackets_for_specials and part.startswith("[") and part.endswith("]"):
            out.append(part.upper() if upper_case_special else part)
        elif word_based:
            out.extend(part.split())
        else:
            out.extend(re.sub(r"\s+", " ", part))
    if word_based:
        return out
    # no blank at the borders, none doubled around specials
    res: List[str] = []
    for s in out:
        if s == " " and (not res or res[-1] == " "):
            continue
        res.append(s)
    while res and res[-1] == " ":
        res.pop()
    return res


def parse_orthography(orthography: str, prefix: Sequence[str] = (), postfix: Sequence[str] = ("[END]",), remove_chars: str = "(){}", collapse_spaces: bool = True,
                      final_strip: bool = True, **kwargs) -> List[str]:
    """:func:`parse_orthography_into_symbols` after removing ``remove_chars``, with prefix and postfix symbols"""
    for c in remove_chars:
        orthography = orthography.replace(c, "")
    if collapse_spaces:
        orthography = " ".join(orthography.split())
    if final_strip:
        orthography = orthography.strip()
    return list(prefix) + parse_orthography_into_symbols(orthography, **kwargs) + list(postfix)


def json_remove_comments(string: str, strip_space: bool = True) -> str:
    """``//`` and ``/* */`` comments out of JSON text (not inside strings)"""
    out, i, n, in_str = [], 0, len(string), False
    while i < n:
        c = string[i]
        if in_str:
            out.append(c)
            if c == "\\" and i + 1 < n:
                out.append(string[i + 1])
                i += 1
            elif c == '"':
                in_str = False
        elif c == '"':
            in_str = True
            out.append(c)
        elif string.startswith("//", i):
            while i < n and string[i] != "\n":
                i += 1
            continue
        elif string.startswith("/*", i):
            j = string.find("*/", i + 2)
            i = n if j < 0 else j + 2
            continue
        else:
            out.append(c)
        i += 1
    res = "".join(out)
    if strip_space:
        res = "\n".join(line.rstrip() for line in res.splitlines() if line.strip())
    return res


# ---- introspection -------------------------------------------------------------------------------------------------------------------
def getargspec(func: Callable):
    """``inspect.getfullargspec``"""
    return inspect.getfullargspec(func)


def collect_class_init_kwargs(cls: type, only_with_default: bool = False) -> List[str]:
    """names of the keyword arguments of ``__init__`` along the MRO (as long as constructors forward ``**kwargs``)"""
    names: List[str] = []
    for c in inspect.getmro(cls):
        init = c.__dict__.get("__init__")
        if init is None or not isinstance(init, types.FunctionType):
            continue
        spec = inspect.getfullargspec(init)
        args = spec.args[1:]
        if only_with_default:
            n_def = len(spec.defaults or ())
            args = args[len(args) - n_def:] if n_def else []
            args += [a for a in spec.kwonlyargs if spec.kwonlydefaults and a in spec.kwonlydefaults]
        else:
            args += spec.kwonlyargs
        for a in args:
            if a not in names:
                names.append(a)
        if spec.varkw is None:
            break
    return names


def collect_mandatory_class_init_kwargs(cls: type) -> List[str]:
    """arguments of ``__init__`` along the MRO that have no default"""
    names: List[str] = []
    for c in inspect.getmro(cls):
        init = c.__dict__.get("__init__")
        if init is None or not isinstance(init, types.FunctionType):
            continue
        spec = inspect.getfullargspec(init)
        args = spec.args[1:]
        n_def = len(spec.defaults or ())
        mandatory = args[: len(args) - n_def] if n_def else args
        mandatory += [a for a in spec.kwonlyargs if not (spec.kwonlydefaults and a in spec.kwonlydefaults)]
        for a in mandatory:
            if a not in names:
                names.append(a)
        if spec.varkw is None:
            break
    return names


def help_on_type_error_wrong_args(cls: type, kwargs: Sequence[str]):
    """after a ``TypeError`` from ``cls(**kwargs)``: print which arguments are unknown or missing"""
    known = set(collect_class_init_kwargs(cls))
    mandatory = set(collect_mandatory_class_init_kwargs(cls))
    unknown = [k for k in kwargs if k not in known]
    missing = [k for k in mandatory if k not in kwargs]
    if unknown:
        print("Args mismatch? Unknown for %s: %r" % (cls.__name__, unknown), file=sys.stderr)
    if missing:
        print("Args mismatch? Missing for %s: %r" % (cls.__name__, sorted(missing)), file=sys.stderr)


def type_attrib_mro_chain(cls: type, attr_name: str) -> List[Any]:
    """the different definitions of an attribute along the MRO, most specific first"""
    out: List[Any] = []
    for c in inspect.getmro(cls):
        if attr_name in c.__dict__ and c.__dict__[attr_name] not in out:
            out.append(c.__dict__[attr_name])
    return out


def next_type_attrib_in_mro_chain(cls: type, attr_name: str, attr: Any) -> Any:
    """the definition that ``attr`` overrides"""
    chain = type_attrib_mro_chain(cls, attr_name)
    return chain[chain.index(attr) + 1]


def generic_import_module(filename: str):
    """import a Python file (``.py``) or a module by dotted name"""
    import importlib
    import importlib.util

    if filename.endswith(".py") or os.sep in filename:
        name = "_imported_" + re.sub(r"\W", "_", os.path.abspath(filename))
        if name in sys.modules:
            return sys.modules[name]
        spec = importlib.util.spec_from_file_location(name, filename)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod
    return importlib.import_module(filename)


class ReportImportedDevModules:
    """callable: prints the packages among the loaded modules that are git checkouts or are named in ``description``"""

    def __init__(self, description: str, mod_names: Sequence[str] = ()):
        self.description = description
        self.mod_names = list(mod_names)

    def __call__(self, file=None):
        file = file or sys.stdout
        for name, mod in sorted(sys.modules.items()):
            if "." in name or mod is None:
                continue
            fn = getattr(mod, "__file__", None)
            if not fn:
                continue
            d = os.path.dirname(os.path.abspath(fn))
            if name in self.mod_names or os.path.isdir(os.path.join(os.path.dirname(d), ".git")) or os.path.isdir(os.path.join(d, ".git")):
                print("%s: module %s from %s" % (self.description, name, d), file=file)


# ---- files, environment, processes ---------------------------------------------------------------------------------------------------
def touch_file(filename: str, mode: int = 0o666):
    """create if missing, set the modification time to now"""
    fd = os.open(filename, os.O_WRONLY | os.O_CREAT, mode)
    os.close(fd)
    os.utime(filename, None)


def maybe_make_dirs(dirname: str):
    """``makedirs`` that tolerates a concurrent creation"""
    os.makedirs(dirname, exist_ok=True)


def get_utc_start_time_filename_part() -> str:
    """start time of this process as ``YYYY-MM-DD-HH-MM-SS``"""
    try:
        import psutil

        t = psutil.Process().create_time()
    except Exception:
        t = time.time()
    return time.strftime("%Y-%m-%d-%H-%M-%S", time.gmtime(t))


def log_runtime_info_to_dir(path: str, config=None):
    """one ``returnn.<start time>.<host>.<pid>.log`` per process in ``path``: command line, versions, environment of the run"""
    import socket

    maybe_make_dirs(path)
    fn = os.path.join(path, "returnn.%s.%s.%i.log" % (get_utc_start_time_filename_part(), socket.gethostname(), os.getpid()))
    lines = ["Start time: %s" % get_utc_start_time_filename_part(), "Call: %s" % sys.argv, "Path: %s" % os.getcwd(), "Hostname: %s" % socket.gethostname(),
             "PID: %i" % os.getpid(), "Version: %s" % describe_returnn_version(), "Torch: %s" % describe_torch_version()]
    if config is not None:
        lines.append("Config files: %s" % getattr(config, "files", None))
    try:
        with open(fn, "w") as f:
            f.write("\n".join(lines) + "\n")
    except OSError as exc:
        print("log_runtime_info_to_dir: %s" % exc, file=sys.stderr)


def cleanup_env_var_path(env_var: str, path_prefix: str):
    """remove the entries under ``path_prefix`` from a ``:``-separated environment variable"""
    if env_var not in os.environ:
        return
    parts = [p for p in os.environ[env_var].split(":") if p and not p.startswith(path_prefix)]
    os.environ[env_var] = ":".join(parts)


def is_valid_fd(fd: int) -> bool:
    """the descriptor is open"""
    try:
        os.fstat(fd)
        return True
    except OSError:
        return False


def close_all_fds_except(except_fds: Iterable[int]):
    """for a freshly forked child: close every descriptor but these (and stdio)"""
    keep = set(except_fds) | {0, 1, 2}
    try:
        fds = [int(x) for x in os.listdir("/proc/self/fd")]
    except OSError:
        fds = list(range(3, 256))
    for fd in fds:
        if fd not in keep:
            try:
                os.close(fd)
            except OSError:
                pass


def read_bytes_to_new_buffer(p, size: int):
    """``size`` bytes from a file object into a fresh ``BytesIO``"""
    import io

    buf = io.BytesIO()
    remaining = size
    while remaining > 0:
        chunk = p.read(remaining)
        if not chunk:
            raise EOFError("expected %i more bytes" % remaining)
        buf.write(chunk)
        remaining -= len(chunk)
    buf.seek(0)
    return buf


def serialize_object(obj: Any) -> bytes:
    """pickle with the pickler that also takes functions and modules of ``__main__`` by value"""
    from .task_system import dumps

    return dumps(obj)


def deserialize_object(s: bytes) -> Any:
    """inverse of :func:`serialize_object`"""
    from .task_system import loads

    return loads(s)


def write_pickled_object(p, obj: Any):
    """length-prefixed pickle onto a binary stream"""
    import struct

    data = serialize_object(obj)
    p.write(struct.pack("<i", len(data)))
    p.write(data)
    p.flush()


def hdf5_dimension(filename: str, dimension: str) -> int:
    """an integer attribute, or the first extent of a dataset, of an HDF file (``h5py`` or the ``.npz`` stand-in)"""
    from .h5_shim import get_h5py

    with get_h5py().File(filename, "r") as f:
        if dimension in f.attrs:
            return int(f.attrs[dimension])
        return int(f[dimension].shape[0])


def hdf5_shape(filename: str, dimension: str) -> Tuple[int, ...]:
    """shape of a dataset of an HDF file"""
    from .h5_shim import get_h5py

    with get_h5py().File(filename, "r") as f:
        return tuple(f[dimension].shape)


def hdf5_group(filename: str, dimension: str) -> Dict[str, Any]:
    """the members of a group as ``{name: first element}``"""
    from .h5_shim import get_h5py

    with get_h5py().File(filename, "r") as f:
        return {k: f[dimension][k][()] if not getattr(f[dimension][k], "shape", ()) else f[dimension][k][0] for k in f[dimension].keys()}


def hdf5_strings(handle, name: str, data: Sequence[str]):
    """store a list of strings as a fixed-width byte-string dataset"""
    arr = numpy.array([s.encode("utf8") for s in data], dtype="S%i" % max([len(s.encode("utf8")) for s in data] + [1]))
    handle.create_dataset(name, data=arr)


def get_patch_atfork_lib() -> Optional[str]:
    """path of the native library that overrides ``pthread_atfork`` (config ``patch_atfork``), None if it was not built"""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    fn = os.path.join(here, "ops", "_build", "librb200_atfork.so")
    return fn if os.path.exists(fn) else None


def restart_returnn():
    """re-execute this process with the same command line"""
    sys.stdout.flush()
    sys.stderr.flush()
    os.execv(sys.executable, [sys.executable] + sys.argv)


def maybe_restart_returnn_with_atfork_patch():
    """if the atfork library exists and is not preloaded yet: preload it and restart"""
    lib = get_patch_atfork_lib()
    if not lib or lib in os.environ.get("LD_PRELOAD", ""):
        return
    os.environ["LD_PRELOAD"] = (os.environ.get("LD_PRELOAD", "") + ":" + lib).lstrip(":")
    restart_returnn()


def overwrite_os_exec(prefix_args: Sequence[str]):
    """every later ``os.exec*`` of this process gets ``prefix_args`` in front of its command line (e.g. a wrapper that sets a library path)"""
    prefix = list(prefix_args)
    orig_execv, orig_execve = os.execv, os.execve

    def execv(path, args):
        if list(args[: len(prefix)]) == prefix:
            return orig_execv(path, args)
        return orig_execv(prefix[0], prefix + list(args))

    def execve(path, args, env):
        if list(args[: len(prefix)]) == prefix:
            return orig_execve(path, args, env)
        return orig_execve(prefix[0], prefix + list(args), env)

    os.execv, os.execve = execv, execve  # type: ignore[assignment]


def collect_proc_maps_exec_files() -> List[str]:
    """files mapped executable into this process (``/proc/self/maps``)"""
    out: List[str] = []
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                parts = line.split(None, 5)
                if len(parts) == 6 and "x" in parts[1] and parts[5].startswith("/"):
                    fn = parts[5].strip()
                    if fn not in out:
                        out.append(fn)
    except OSError:
        pass
    return out


def find_libcudart_from_runtime() -> Optional[str]:
    """the CUDA runtime library mapped into this process, if any"""
    for fn in collect_proc_maps_exec_files():
        if re.match(r".*/libcudart\.so(\.[0-9.]+)?$", fn):
            return fn
    return None
