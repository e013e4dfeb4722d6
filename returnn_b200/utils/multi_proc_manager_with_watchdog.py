"""
``multiprocessing`` SyncManager whose server process exits when the parent process dies (a watchdog thread polls the
parent pid), so that no orphaned manager processes stay behind after a crash.

Parity: returnn/util/multi_proc_manager_with_watchdog.py:20-64.
"""

from __future__ import annotations
import multiprocessing.managers
import os
import threading
import time


def _watchdog(parent_pid: int):
    def loop():
        while True:
            time.sleep(1.0)
            if os.getppid() != parent_pid:
                os._exit(1)

    threading.Thread(target=loop, name="manager-watchdog", daemon=True).start()


def create_manager() -> multiprocessing.managers.SyncManager:
    """started SyncManager with watchdog"""
    manager = multiprocessing.managers.SyncManager(ctx=multiprocessing.get_context("spawn"))
    manager.start(initializer=_watchdog, initargs=(os.getpid(),))
    return manager
