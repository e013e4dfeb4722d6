"""
Loader of the small native helper library (``librb200_host.so``: signal handler with C backtrace, ``pthread_atfork``
patch, Python-literal-to-pickle parser), built in-tree by :mod:`returnn_b200.ops.build` with g++ (no CUDA needed).

Parity: returnn/util/debug.py:283-345 (signal handler), returnn/util/basic.py:3895-3950 (atfork patch),
returnn/util/py-to-pickle.cpp + literal_py_to_pickle.py.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import os
import sys

_HOST_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ops", "_build", "librb200_host.so")
_ATFORK_LIB = os.path.join(os.path.dirname(_HOST_LIB), "librb200_atfork.so")
_lib = None
_tried = False


def get_native_lib() -> Optional[ctypes.CDLL]:
    """the host helper library or None"""
    global _lib, _tried
    if not _tried:
        _tried = True
        if os.path.exists(_HOST_LIB):
            _lib = ctypes.CDLL(_HOST_LIB)
    return _lib


def maybe_restart_with_atfork_patch():
    """re-exec the process with the atfork patch library preloaded (config ``patch_atfork``)"""
    if os.environ.get("__RETURNN_ATFORK_PATCHED") == "1":
        return
    if not os.path.exists(_ATFORK_LIB):
        print("patch_atfork: %s not built, ignoring" % _ATFORK_LIB, file=sys.stderr)
        return
    env = os.environ.copy()
    env["LD_PRELOAD"] = _ATFORK_LIB + ((":" + env["LD_PRELOAD"]) if env.get("LD_PRELOAD") else "")
    env["__RETURNN_ATFORK_PATCHED"] = "1"
    os.execvpe(sys.executable, [sys.executable] + sys.argv, env)
