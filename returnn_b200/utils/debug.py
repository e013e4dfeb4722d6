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


def init_better_exchook():
    """the extended exception hook for the main thread and all threads"""
    from . import better_exchook

    better_exchook.install()


def format_signum(signum: int) -> str:
    """``11 (SIGSEGV)``"""
    import signal

    try:
        return "%i (%s)" % (signum, signal.Signals(signum).name)
    except ValueError:
        return "%i (unknown)" % signum


def signal_handler(signum, frame):
    """prints the stacks of all threads, then re-raises the signal with the default action"""
    import os
    import signal
    import sys

    print("Signal handler: got signal %s" % format_signum(signum), file=sys.stderr)
    dump_all_thread_tracebacks(file=sys.stderr)
    signal.signal(signum, signal.SIG_DFL)
    os.kill(os.getpid(), signum)


def install_signal_handler_if_default(signum: int, exceptions_are_fatal: bool = False) -> bool:
    """:func:`signal_handler` for ``signum`` unless a handler other than the default is installed already"""
    import signal

    try:
        if signal.getsignal(signum) == signal.SIG_DFL:
            signal.signal(signum, signal_handler)
            return True
    except Exception:
        if exceptions_are_fatal:
            raise
    return False


def install_lib_sig_segfault():
    """the native handler that prints a C-level backtrace on SIGSEGV / SIGBUS / SIGILL / SIGFPE / SIGABRT"""
    return install_native_signal_handler()


def setup_warn_with_traceback():
    """every ``warnings.warn`` prints the Python stack of its origin"""
    import sys
    import traceback
    import warnings

    def warn_with_traceback(message, category, filename, lineno, file=None, line=None):
        out = file if file is not None and hasattr(file, "write") else sys.stderr
        traceback.print_stack(file=out)
        out.write(warnings.formatwarning(message, category, filename, lineno, line))

    warnings.showwarning = warn_with_traceback


def init_cuda_not_in_main_proc_check():
    """after this, initialising CUDA in this process raises (for a parent that must leave the GPUs to its children)"""
    import torch

    def _refuse(*_a, **_kw):
        raise RuntimeError("CUDA must not be initialised in this process (init_cuda_not_in_main_proc_check)")

    torch.cuda._lazy_init = _refuse  # type: ignore[assignment]


def init_ipython_kernel():
    """an IPython kernel in a background thread to attach to the running process (needs ``ipykernel``)"""
    try:
        import ipykernel.kernelapp  # noqa: F401
    except ImportError:
        print("init_ipython_kernel: ipykernel is not installed")
        return
    import threading
    from ipykernel.kernelapp import IPKernelApp

    def run():
        app = IPKernelApp.instance()
        app.initialize([])
        app.start()

    threading.Thread(target=run, name="IPython kernel", daemon=True).start()
