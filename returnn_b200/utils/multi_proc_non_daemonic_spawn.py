"""
A multiprocessing "spawn" context whose processes are not daemonic (so they may start their own child processes,
e.g. a DataLoader worker whose dataset is a MultiProcDataset) and that runs a picklable pre-init function in the
child before the target (to install the global config). Children are terminated when the parent exits.

Parity: returnn/util/multi_proc_non_daemonic_spawn.py:51-192.
"""

from __future__ import annotations
from typing import Any, Callable, Optional
import atexit
import multiprocessing
import multiprocessing.context
import os
import signal
import sys
import weakref

_live_procs = weakref.WeakSet()
_atexit_registered = False


def _cleanup_children():
    for p in list(_live_procs):
        try:
            if p.is_alive():
                p.terminate()
        except Exception:
            pass
    for p in list(_live_procs):
        try:
            p.join(timeout=1)
            if p.is_alive():
                p.kill()
        except Exception:
            pass


class _PreInitTarget:
    def __init__(self, pre_init: Optional[Callable[[], None]], target, parent_pid: int):
        self.pre_init = pre_init
        self.target = target
        self.parent_pid = parent_pid

    def __call__(self, *args, **kwargs):
        try:
            # die with the parent
            import ctypes

            libc = ctypes.CDLL(None)
            libc.prctl(1, signal.SIGTERM)  # PR_SET_PDEATHSIG
            if os.getppid() != self.parent_pid:
                sys.exit(1)
        except Exception:
            pass
        if self.pre_init is not None:
            self.pre_init()
        if self.target is not None:
            return self.target(*args, **kwargs)


class NonDaemonicSpawnProcess(multiprocessing.context.SpawnProcess):
    """spawned process which reports daemon=False"""

    _pre_init_func: Optional[Callable[[], None]] = None

    def __init__(self, group=None, target=None, name=None, args=(), kwargs=None, *, daemon=None, pre_init_func=None):
        global _atexit_registered
        target = _PreInitTarget(pre_init_func or self._pre_init_func, target, os.getpid())
        super().__init__(group=group, target=target, name=name, args=args, kwargs=kwargs or {}, daemon=False)
        if not _atexit_registered:
            atexit.register(_cleanup_children)
            _atexit_registered = True

    @property
    def daemon(self):
        """never daemonic"""
        return False

    @daemon.setter
    def daemon(self, value):
        pass

    def start(self):
        super().start()
        _live_procs.add(self)


class NonDaemonicSpawnContext(multiprocessing.context.SpawnContext):
    """spawn context creating :class:`NonDaemonicSpawnProcess`"""

    def __init__(self, *, process_pre_init_func: Optional[Callable[[], None]] = None):
        super().__init__()
        self.process_pre_init_func = process_pre_init_func

        class _Process(NonDaemonicSpawnProcess):
            _pre_init_func = process_pre_init_func

        _Process.__name__ = "NonDaemonicSpawnProcess"
        _Process.__qualname__ = "NonDaemonicSpawnProcess"
        self._process_cls = _Process

    def Process(self, *args, **kwargs):
        """create process"""
        kwargs.setdefault("pre_init_func", self.process_pre_init_func)
        return NonDaemonicSpawnProcess(*args, **kwargs)
