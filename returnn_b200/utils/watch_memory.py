"""
Background process that reports the memory of the main process and all its (grand)children whenever the set of processes
or the total changes noticeably. Helps to find which dataset worker grows.

Parity: returnn/util/watch_memory.py (watch_memory :19, get_mem_info :133).
"""

from __future__ import annotations
from typing import Dict
import os
import time


def watch_memory():
    """start the watcher (a non-daemonic spawned process that exits with its parent)"""
    from .multi_proc_non_daemonic_spawn import NonDaemonicSpawnContext

    ctx = NonDaemonicSpawnContext(process_pre_init_func=None)
    proc = ctx.Process(target=_watch_main, args=(os.getpid(),), name="watch_memory", daemon=True)
    proc.start()
    return proc


def _fmt_size(c: int) -> str:
    for unit, f in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if c >= f:
            return "%.1f%s" % (c / f, unit)
    return "%iB" % c


def get_mem_info(proc) -> Dict[str, int]:
    """:return: rss / pss / uss / shared where the platform provides them"""
    try:
        info = proc.memory_full_info()
    except Exception:
        info = proc.memory_info()
    res = {}
    for k in ("rss", "pss", "uss", "shared"):
        if hasattr(info, k):
            res[k] = int(getattr(info, k))
    return res


def _watch_main(pid: int, *, interval: float = 5.0, rel_change: float = 0.05):
    import psutil

    try:
        main = psutil.Process(pid)
    except psutil.NoSuchProcess:
        return
    last_total = -1
    last_pids = set()
    while True:
        try:
            if not main.is_running():
                return
            procs = [main] + main.children(recursive=True)
        except psutil.NoSuchProcess:
            return
        procs = [p for p in procs if p.pid != os.getpid()]
        infos = {}
        for p in procs:
            try:
                infos[p.pid] = (p.name(), get_mem_info(p))
            except (psutil.NoSuchProcess, psutil.AccessDenied):
                pass
        total = sum(i.get("pss", i.get("rss", 0)) for _, i in infos.values())
        pids = set(infos.keys())
        if pids != last_pids or last_total < 0 or abs(total - last_total) > rel_change * max(last_total, 1):
            print("MEMORY: total (main %i + %i children) %s" % (pid, len(pids) - 1, _fmt_size(total)))
            for q, (name, i) in sorted(infos.items()):
                if q not in last_pids or len(infos) <= 8:
                    print("MEMORY:   %s(%i) %s" % (name, q, " ".join("%s=%s" % (k, _fmt_size(v)) for k, v in i.items())))
            last_total, last_pids = total, pids
        time.sleep(interval)
