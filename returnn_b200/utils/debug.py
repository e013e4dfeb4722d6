"""
Debugging helpers: fault handlers (Python ``faulthandler`` plus a native handler that prints a C backtrace on
SIGSEGV/SIGBUS/SIGILL/SIGABRT/SIGFPE and a thread dump on SIGUSR1), thread stack dumps, an interactive debug shell.

Parity: returnn/util/debug.py (init_faulthandler, native signal handler :283-345, dump_all_thread_tracebacks, debug_shell).
"""

from __future__ import annotations
from typing import Any, Dict, Optional
import os
import signal
import sys
import threading
import traceback


def dump_all_thread_tracebacks(*, exclude_thread_ids=None, exclude_self: bool = False, file=None):
    """print the Python stack of every thread"""
    if file is None:
        file = sys.stdout
    exclude = set(exclude_thread_ids or [])
    if exclude_self:
        exclude.add(threading.get_ident())
    names = {t.ident: t.name for t in threading.enumerate()}
    for tid, frame in sys._current_frames().items():
        if tid in exclude:
            continue
        print("Thread %s (%s):" % (names.get(tid, "?"), tid), file=file)
        for line in traceback.format_stack(frame):
            file.write(line)
        print(file=file)


def _sigusr1_handler(sig, frame):
    print("Got SIGUSR1, dumping all threads:", file=sys.stderr)
    dump_all_thread_tracebacks(file=sys.stderr)


def install_native_signal_handler() -> bool:
    """load the native handler library (C backtrace on fatal signals); False if it is not built"""
    from .native_helpers import get_native_lib

    lib = get_native_lib()
    if lib is None or not hasattr(lib, "rb200_install_signal_handler"):
        return False
    lib.rb200_install_signal_handler()
    return True


def init_faulthandler(sigusr1_chain: bool = False):
    """install faulthandler, the native handler, and the SIGUSR1 thread dump"""
    import faulthandler

    try:
        faulthandler.enable()
    except Exception:
        pass
    if os.environ.get("RETURNN_NATIVE_SIGNAL_HANDLER", "1") == "1":
        try:
            install_native_signal_handler()
        except Exception:
            pass
    if hasattr(signal, "SIGUSR1") and threading.current_thread() is threading.main_thread():
        try:
            if sigusr1_chain:
                faulthandler.register(signal.SIGUSR1, all_threads=True, chain=True)
            else:
                signal.signal(signal.SIGUSR1, _sigusr1_handler)
        except (ValueError, OSError):
            pass


def debug_shell(user_ns: Optional[Dict[str, Any]] = None, user_global_ns: Optional[Dict[str, Any]] = None, exit_afterwards: bool = True):
    """interactive shell (IPython if available)"""
    print("Debug shell:")
    ns = dict(user_global_ns or {})
    ns.update(user_ns or {})
    try:
        import IPython

        IPython.embed(user_ns=ns)
    except ImportError:
        import code

        code.interact(local=ns)
    if exit_afterwards:
        print("Debug shell exit. Exit now.")
        sys.exit(1)


class PyTracer:
    """
    Trace local variable values of given functions while a block runs: ``with PyTracer([fn], Tensor) as t: ...``;
    afterwards ``t.captured_locals[fn]`` lists per call the dict name -> list of values of the given types.
    """

    def __init__(self, funcs_to_trace_list, capture_type):
        self.funcs = list(funcs_to_trace_list)
        self.capture_type = capture_type
        self.captured_locals: Dict[Any, list] = {}
        self._codes = {getattr(f, "__code__", None): f for f in self.funcs}
        self._prev = None

    def __enter__(self):
        self._prev = sys.gettrace()
        sys.settrace(self._trace)
        return self

    def __exit__(self, *a):
        sys.settrace(self._prev)

    def _trace(self, frame, event, arg):
        func = self._codes.get(frame.f_code)
        if func is None:
            return self._trace if self._prev is None else self._prev
        if event == "call":
            self.captured_locals.setdefault(func, []).append({})
        elif event in ("line", "return"):
            cur = self.captured_locals[func][-1]
            for k, v in frame.f_locals.items():
                if isinstance(v, self.capture_type):
                    lst = cur.setdefault(k, [])
                    if not lst or lst[-1] is not v:
                        lst.append(v)
        return self._trace
