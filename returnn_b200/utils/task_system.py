"""
Moving Python objects between processes when the standard pickler cannot: functions and classes that live in a config file
(a module that the other process cannot import by name), lambdas, closures, bound methods, and large numpy arrays.

:class:`Pickler` extends :class:`pickle.Pickler` through ``reducer_override``:

* a function that cannot be found again under ``module.qualname`` is sent by value: its code object (``marshal``), defaults,
  closure cells, and the subset of its globals that the code names; the globals of all functions from one module are rebuilt
  as ONE shared dict on the other side, so functions that call each other (or share module state) keep doing so;
* classes defined in such a module are sent as ``type(name, bases, dict)``;
* modules are sent by name;
* numpy arrays above a size threshold can travel through POSIX shared memory (:class:`SharedNumpyArray`) instead of the pipe.

``dumps`` / ``loads`` are the convenience pair. The reference has the same role in returnn/util/task_system.py:571 (Pickler) and
:128 (SharedNumpyArray); the dataset worker processes (returnn/datasets/postprocessing.py:817) are the user.
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Tuple
import importlib
import io
import marshal
import pickle
import sys
import types
import numpy

__all__ = ["Pickler", "Unpickler", "dumps", "loads", "SharedNumpyArray", "use_shared_mem_for_numpy_array", "next_power_of_two"]


def next_power_of_two(n: int) -> int:
    """smallest power of two >= n"""
    return 1 << max(int(n) - 1, 0).bit_length()


# ---------------------------------------------------------------------------------------------------------------------
# shared-memory numpy arrays


class SharedNumpyArray:
    """
    A numpy array whose storage is a named shared-memory block. Pickling sends (name, shape, dtype) only; the receiver
    maps the same block. The creator owns the block and unlinks it in :func:`close` (or when collected); receivers only detach.
    """

    def __init__(self, shape, dtype, *, _name: Optional[str] = None, _untrack: bool = True):
        from multiprocessing import shared_memory

        self.shape = tuple(int(d) for d in shape)
        self.dtype = numpy.dtype(dtype)
        nbytes = max(int(numpy.prod(self.shape, dtype=numpy.int64)) * self.dtype.itemsize, 1)
        if _name is None:
            self._shm = shared_memory.SharedMemory(create=True, size=nbytes)
            self._owner = True
        else:
            self._shm = shared_memory.SharedMemory(name=_name)
            self._owner = False
            if _untrack:
                self._untrack()  # this process's resource tracker must not unlink the creator's block at exit
        self.array = numpy.ndarray(self.shape, dtype=self.dtype, buffer=self._shm.buf)

    def _untrack(self):
        try:
            from multiprocessing import resource_tracker

            resource_tracker.unregister(self._shm._name, "shared_memory")  # noqa
        except Exception:
            pass

    @classmethod
    def from_array(cls, arr: numpy.ndarray) -> "SharedNumpyArray":
        """copy ``arr`` into a new block"""
        out = cls(arr.shape, arr.dtype)
        out.array[...] = arr
        return out

    @property
    def name(self) -> str:
        """name of the block"""
        return self._shm.name

    def __reduce__(self):
        return _attach_shared, (self._shm.name, self.shape, self.dtype.str)

    def close(self):
        """detach; the creator also removes the block"""
        shm, self._shm = self._shm, None
        if shm is None:
            return
        self.array = None
        try:
            shm.close()
        except BufferError:
            pass  # a view is still alive somewhere; the mapping goes away with it
        if self._owner:
            try:
                shm.unlink()
            except FileNotFoundError:
                pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _attach_shared(name: str, shape, dtype_str: str) -> SharedNumpyArray:
    return SharedNumpyArray(shape, dtype_str, _name=name)


_SHARED_MIN_BYTES = 1 << 20


def use_shared_mem_for_numpy_array(obj: numpy.ndarray, min_bytes: int = _SHARED_MIN_BYTES) -> bool:
    """whether ``Pickler(shared_mem=True)`` sends this array through shared memory"""
    return isinstance(obj, numpy.ndarray) and obj.dtype != object and obj.nbytes >= min_bytes


def _array_from_shared(name: str, shape, dtype_str: str) -> numpy.ndarray:
    """receiver side: copy out of the block and release it (the sender passed ownership along)"""
    sh = SharedNumpyArray(shape, dtype_str, _name=name, _untrack=False)  # tracked here: this side removes it
    out = numpy.array(sh.array, copy=True)
    sh._owner = True  # the block was made for this one transfer
    sh.close()
    return out


# ---------------------------------------------------------------------------------------------------------------------
# functions and classes by value

_by_value_globals: Dict[str, Dict[str, Any]] = {}  # receiver side: one globals dict per sending module


def _importable(obj, module_name: Optional[str], qualname: str) -> bool:
    """whether ``module_name.qualname`` gives back exactly ``obj`` in a fresh interpreter (approximated in this one)"""
    if not module_name or module_name == "__main__":
        return False
    mod = sys.modules.get(module_name)
    if mod is None:
        return False
    if getattr(mod, "__file__", None) is None and getattr(mod, "__spec__", None) is None and module_name not in sys.builtin_module_names:
        return False  # a module object without a file (a config run through exec) cannot be imported elsewhere
    cur = mod
    for part in qualname.split("."):
        if part == "<locals>" or part == "<lambda>":
            return False
        cur = getattr(cur, part, None)
        if cur is None:
            return False
    return cur is obj


def _names_of_code(code: types.CodeType):
    names = set(code.co_names)
    for const in code.co_consts:
        if isinstance(const, types.CodeType):
            names |= _names_of_code(const)
    return names


def _make_cell(value=None, empty: bool = False):
    if empty:
        return types.CellType()
    return types.CellType(value)


def _rebuild_function(code_bytes: bytes, module_key: str, name: str, qualname: str, defaults, kwdefaults, closure, fdict, annotations, doc):
    code = marshal.loads(code_bytes)
    g = _by_value_globals.setdefault(module_key, {"__builtins__": __builtins__, "__name__": module_key})
    func = types.FunctionType(code, g, name, defaults, closure)
    func.__qualname__ = qualname
    func.__kwdefaults__ = kwdefaults
    func.__module__ = module_key
    if annotations:
        func.__annotations__ = annotations
    func.__doc__ = doc
    if fdict:
        func.__dict__.update(fdict)
    return func


def _set_function_globals(func: types.FunctionType, needed: Dict[str, Any]):
    """second step (after the function object exists, so that recursion and mutual references work)"""
    for k, v in needed.items():
        func.__globals__.setdefault(k, v)
    return func


def _rebuild_class(module_key: str, name: str, qualname: str, bases, cls_dict: Dict[str, Any]):
    g = _by_value_globals.setdefault(module_key, {"__builtins__": __builtins__, "__name__": module_key})
    existing = g.get("__class__:" + qualname)
    if existing is not None:
        return existing
    cls_dict = dict(cls_dict)
    cls_dict["__module__"] = module_key
    cls = type(name, bases, cls_dict)
    cls.__qualname__ = qualname
    g["__class__:" + qualname] = cls
    return cls


def _import_module(name: str):
    return importlib.import_module(name)


class Pickler(pickle.Pickler):
    """see the module docstring"""

    def __init__(self, file, protocol: int = pickle.HIGHEST_PROTOCOL, *, shared_mem: bool = False, shared_mem_min_bytes: int = _SHARED_MIN_BYTES):
        super().__init__(file, protocol)
        self.shared_mem = shared_mem
        self.shared_mem_min_bytes = shared_mem_min_bytes
        self._in_progress: Dict[int, Any] = {}

    def reducer_override(self, obj):  # noqa: C901
        """by-value forms for what the standard pickler would refuse or send by a name that does not resolve elsewhere"""
        if isinstance(obj, types.FunctionType):
            if _importable(obj, getattr(obj, "__module__", None), obj.__qualname__):
                return NotImplemented
            return self._reduce_function(obj)
        if isinstance(obj, types.ModuleType):
            return _import_module, (obj.__name__,)
        if isinstance(obj, types.CodeType):
            return marshal.loads, (marshal.dumps(obj),)
        if isinstance(obj, types.CellType):
            try:
                return _make_cell, (obj.cell_contents,)
            except ValueError:
                return _make_cell, (None, True)
        if isinstance(obj, type):
            if obj.__module__ in ("builtins",) or _importable(obj, obj.__module__, obj.__qualname__):
                return NotImplemented
            return self._reduce_class(obj)
        if self.shared_mem and isinstance(obj, numpy.ndarray) and use_shared_mem_for_numpy_array(obj, self.shared_mem_min_bytes):
            sh = SharedNumpyArray.from_array(obj)
            sh._owner = False  # ownership travels with the message
            sh._untrack()
            name, shape, dt = sh.name, sh.shape, sh.dtype.str
            sh.close()
            return _array_from_shared, (name, shape, dt)
        if isinstance(obj, (io.BufferedReader, io.BufferedWriter, io.TextIOWrapper)):
            return _none, ()  # open files do not travel
        return NotImplemented

    def _reduce_function(self, func: types.FunctionType):
        code = func.__code__
        module_key = func.__module__ or "__by_value__"
        needed = {}
        g = func.__globals__
        for name in _names_of_code(code):
            if name in g and name != "__builtins__":
                needed[name] = g[name]
        closure = func.__closure__
        fdict = {k: v for k, v in func.__dict__.items()} or None
        args = (marshal.dumps(code), module_key, func.__name__, func.__qualname__, func.__defaults__, func.__kwdefaults__, closure,
                fdict, None, func.__doc__)
        # (callable, args, state, listitems, dictitems, state_setter): the state step fills in the globals after the function
        # object is memoised, so that self-reference and mutual recursion terminate
        return _rebuild_function, args, needed, None, None, _set_function_globals

    def _reduce_class(self, cls: type):
        skip = {"__dict__", "__weakref__", "__module__", "__qualname__"}
        cls_dict = {k: v for k, v in vars(cls).items() if k not in skip and not isinstance(v, (types.GetSetDescriptorType, types.MemberDescriptorType))}
        return _rebuild_class, (cls.__module__ or "__by_value__", cls.__name__, cls.__qualname__, cls.__bases__, cls_dict)


def _none():
    return None


Unpickler = pickle.Unpickler


def dumps(obj, *, shared_mem: bool = False) -> bytes:
    """object -> bytes"""
    buf = io.BytesIO()
    Pickler(buf, shared_mem=shared_mem).dump(obj)
    return buf.getvalue()


def loads(data: bytes):
    """bytes -> object"""
    return pickle.loads(data)
