"""
Fast ``literal_eval`` for big data files: the native parser turns Python literal text into pickle bytes which
``pickle.loads`` then materialises (reference: returnn/util/literal_py_to_pickle.py:16-80, py-to-pickle.cpp).
Falls back to ``ast.literal_eval`` when the helper library is not built or the input uses syntax the parser rejects.
"""

from __future__ import annotations
from typing import Any, Union
import ast
import ctypes
import pickle
from .native_helpers import get_native_lib


def literal_eval(text: Union[str, bytes]) -> Any:
    """value of the literal"""
    raw = text.encode("utf8") if isinstance(text, str) else bytes(text)
    lib = get_native_lib()
    if lib is not None and hasattr(lib, "rb200_py_to_pickle"):
        try:
            return pickle.loads(py_to_pickle(raw))
        except ValueError:
            pass
    return ast.literal_eval(raw.decode("utf8"))


def py_to_pickle(raw: bytes) -> bytes:
    """pickle bytes of the literal; raises ValueError with the parser's message"""
    lib = get_native_lib()
    if lib is None or not hasattr(lib, "rb200_py_to_pickle"):
        raise RuntimeError("native helper library not built (python -m returnn_b200.ops.build)")
    fn = lib.rb200_py_to_pickle
    fn.restype = ctypes.c_void_p
    fn.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.POINTER(ctypes.c_longlong), ctypes.c_char_p, ctypes.c_int]
    out_len = ctypes.c_longlong(0)
    err = ctypes.create_string_buffer(256)
    ptr = fn(raw, len(raw), ctypes.byref(out_len), err, 256)
    if not ptr:
        raise ValueError("py_to_pickle: %s" % err.value.decode("utf8", "replace"))
    try:
        return ctypes.string_at(ptr, out_len.value)
    finally:
        lib.rb200_py_to_pickle_free.argtypes = [ctypes.c_void_p]
        lib.rb200_py_to_pickle_free(ptr)
