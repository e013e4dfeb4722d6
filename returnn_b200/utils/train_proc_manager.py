"""
Training process manager: a parent process that (re)starts the training until the final epoch exists or a run makes no
progress. A crash (OOM of the host, a lost device, a preempted node) then costs at most one epoch.

Parity: returnn/util/train_proc_manager.py (maybe_start_train_proc_manager :18, main_proc_manager :39).
"""

from __future__ import annotations
import os
import subprocess
import sys
import time

_ENV_FLAG = "__RETURNN_B200_PROC_MANAGED"


def maybe_start_train_proc_manager(*, config):
    """become the manager when ``task == "train"``, ``start_epoch == "auto"``, single process; returns in the managed child"""
    if os.environ.get(_ENV_FLAG) == "1":
        print("Running in managed mode.")
        return
    if config.value("task", "train") != "train" or config.value("start_epoch", "auto") != "auto":
        return
    if config.typed_value("torch_distributed") is not None or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return  # the launcher of the ranks owns restarts
    main_proc_manager(config=config)


def main_proc_manager(*, config):
    """runs in the parent; never returns (``sys.exit`` with the last return code)"""
    from ..engine.base import EngineBase
    from .basic import hms

    os.environ[_ENV_FLAG] = "1"
    print("train proc manager starting, pid %i" % os.getpid())
    final_epoch = EngineBase.config_get_final_epoch(config)
    t0 = time.time()
    starts = 0
    prev_epoch = None
    rc = None
    while True:
        models = EngineBase.get_existing_models(config, for_training=True)
        cur = max(models) if models else 0
        print("Most recent trained model epoch: %i (%s)" % (cur, models.get(cur)))
        if cur >= final_epoch:
            print("Already finished, nothing to do" if rc is None else ("Finished training" if rc == 0 else "Finished training, last return code %i" % rc))
            rc = 0 if rc is None else rc
            break
        if prev_epoch is not None:
            print("-> trained %i epoch(s) in the last run" % (cur - prev_epoch))
            if cur == prev_epoch:
                print("-> no progress, giving up")
                break
            print("Restarting...")
        prev_epoch = cur
        starts += 1
        t1 = time.time()
        args = [sys.executable] + sys.argv
        print("Run %r" % (args,))
        sys.stdout.flush()
        rc = subprocess.call(args)
        print("runtime %s, return code %i" % (hms(time.time() - t1), rc))
    print("Total starts: %i, total runtime %s" % (starts, hms(time.time() - t0)))
    sys.exit(rc if rc is not None else -1)
