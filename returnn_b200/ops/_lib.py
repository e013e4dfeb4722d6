"""
Loader of the native kernel library (``librb200.so``, built in-tree by :mod:`returnn_b200.ops.build`).

All kernels are exported as plain C functions taking raw device pointers, sizes and a CUDA stream; the Python
wrappers pass ``tensor.data_ptr()`` and the current torch stream, so launches are ordered with torch work and are
capturable into CUDA graphs.

Policy on a machine with a GPU: a missing library is an error (set ``RETURNN_B200_ALLOW_TORCH_FALLBACK=1`` to run the
torch reference implementations instead). On CPU-only machines the torch implementations are always used.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import os
import threading

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build")
_LIB_PATH = os.path.join(_LIB_DIR, "librb200.so")
_lib: Optional[ctypes.CDLL] = None
_lib_tried = False
_lock = threading.Lock()


class NativeLibMissing(RuntimeError):
    """the sm_100a kernel library is not built"""


def lib_path() -> str:
    """where the library is expected"""
    return _LIB_PATH


def get_lib(required: bool = False) -> Optional[ctypes.CDLL]:
    """:return: the loaded library or None"""
    global _lib, _lib_tried
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None and not _lib_tried:
            _lib_tried = True
            if os.path.exists(_LIB_PATH):
                _lib = ctypes.CDLL(_LIB_PATH)
                _declare(_lib)
    if _lib is None and required:
        raise NativeLibMissing(
            "native kernel library not found at %s; run `python -m returnn_b200.ops.build`" % _LIB_PATH)
    return _lib


def allow_fallback() -> bool:
    """env switch to allow torch implementations on GPU"""
    return os.environ.get("RETURNN_B200_ALLOW_TORCH_FALLBACK", "0") == "1"


def use_native(*tensors) -> bool:
    """
    Decide whether the native kernels handle these tensors: all on CUDA, and the library is there.
    On CUDA without the library: error unless the fallback is allowed.
    """
    import torch

    if not tensors or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in tensors if t is not None):
        return False
    if _env_data.get(b"RETURNN_B200_DISABLE_NATIVE", b"0") == b"1":  # read on every call (tests toggle it), without the str encode
        return False
    lib = get_lib()
    if lib is None:
        if allow_fallback():
            return False
        raise NativeLibMissing(
            "CUDA tensors but the sm_100a kernel library is missing (%s). Build it with `python -m returnn_b200.ops.build` "
            "or set RETURNN_B200_ALLOW_TORCH_FALLBACK=1." % _LIB_PATH)
    return True


_env_data = getattr(os.environ, "_data", None)
if not isinstance(_env_data, dict) or (_env_data and not isinstance(next(iter(_env_data)), bytes)):

    class _EnvBytes:
        """fallback where os.environ has no bytes-keyed dict behind it"""

        @staticmethod
        def get(key: bytes, default: bytes) -> bytes:
            return os.environ.get(key.decode(), default.decode()).encode()

    _env_data = _EnvBytes()


def stream_ptr() -> int:
    """current torch CUDA stream as integer handle"""
    import torch

    # the raw handle without the Stream object (current_stream() costs ~15 us of Python per call; a step makes hundreds)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_launch_count = 0


def count_launch(n: int = 1):
    """bookkeeping of native kernel launches (bench reports it)"""
    global _launch_count
    _launch_count += n


def launch_count() -> int:
    """number of native kernel launches so far"""
    return _launch_count


def check(status: int, what: str):
    """raise on a non-zero status returned by a native entry point"""
    if status != 0:
        lib = get_lib()
        msg = ""
        if lib is not None and hasattr(lib, "rb200_last_error"):
            lib.rb200_last_error.restype = ctypes.c_char_p
            m = lib.rb200_last_error()
            msg = m.decode() if m else ""
        raise RuntimeError("%s failed with status %i %s" % (what, status, msg))


def _declare(lib: ctypes.CDLL):
    """every entry point returns an int status; argument types are declared by the wrapper modules"""
    return


def bind(name: str, argtypes):
    """look up an entry point and set its signature (idempotent)"""
    lib = get_lib(required=True)
    fn = getattr(lib, name)
    if getattr(fn, "_rb_bound", False) is not True:
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
        fn._rb_bound = True
    return fn
