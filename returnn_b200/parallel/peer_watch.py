"""
Host-side liveness of the ranks of a data-parallel job.

A collective whose peer has died does not return: NCCL waits for its process-group timeout (half an hour by default), our own
NVLink kernels give up after their bounded spin and report a status word. Both are the expensive way to learn of a failure.
The cheap way is to ask on the host BEFORE the next launch: every rank writes a heartbeat (step number and wall time) into
the key-value store that the process group was set up with, from a daemon thread, and marks itself as "left" when it leaves
on purpose between two steps; the engine checks the peers' entries before it issues a step and raises :class:`PeerFailure`
instead of entering a collective that cannot complete. The training process manager (``use_train_proc_manager``) then
restarts from the last checkpoint.

Config: ``torch_distributed = {..., "peer_watch": {"interval_sec": 0.5, "max_age_sec": 10.0}}`` (or ``True`` for the defaults).

No device code is involved: nothing here waits on a GPU, and a rank only ever leaves between steps, when none of its kernels
or collectives is in flight.

The reference has no counterpart; its failure handling is the NCCL timeout plus returnn/util/train_proc_manager.py.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional
import threading
import time


class PeerFailure(RuntimeError):
    """a peer rank left the job or stopped sending heartbeats; ``ranks`` lists them"""

    def __init__(self, ranks: List[int], reasons: Dict[int, str]):
        self.ranks = list(ranks)
        self.reasons = dict(reasons)
        super().__init__("ranks %s are gone (%s)" % (self.ranks, ", ".join("%i: %s" % (r, reasons[r]) for r in self.ranks)))


class PeerWatch:
    """heartbeats through a ``torch.distributed`` store (any object with ``set(key, str)`` and ``get(key) -> bytes``)"""

    def __init__(self, store, *, rank: int, world: int, interval_sec: float = 0.5, max_age_sec: float = 10.0, prefix: str = "rb200/alive",
                 clock=time.time, start_thread: bool = True):
        """
        :param store: e.g. ``torch.distributed.distributed_c10d._get_default_store()`` or a ``TCPStore``
        :param interval_sec: period of the heartbeat thread
        :param max_age_sec: a peer whose last heartbeat is older than this counts as failed
        :param clock: wall clock (the ranks of one node share it; across nodes the clocks must agree to within max_age_sec)
        :param start_thread: False: the owner calls :func:`beat` itself (tests)
        """
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.interval_sec, self.max_age_sec, self.prefix = float(interval_sec), float(max_age_sec), prefix
        self._clock = clock
        self._step = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.beat()
        if start_thread:
            self._thread = threading.Thread(target=self._run, name="peer-watch-heartbeat", daemon=True)
            self._thread.start()

    def _key(self, rank: int) -> str:
        return "%s/%i" % (self.prefix, rank)

    def _run(self):
        while not self._stop.wait(self.interval_sec):
            try:
                self.beat()
            except Exception:
                return  # the store is gone: the job is ending

    def beat(self, step: Optional[int] = None):
        """write this rank's heartbeat"""
        if step is not None:
            self._step = int(step)
        self.store.set(self._key(self.rank), "alive:%i:%.3f" % (self._step, self._clock()))

    def leave(self, reason: str = "left"):
        """this rank leaves on purpose (call it between steps, after a device synchronisation); stops the heartbeat"""
        self._stop.set()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=2 * self.interval_sec + 1.0)
        self.store.set(self._key(self.rank), "left:%s" % reason)

    def close(self):
        """stop the heartbeat thread without marking the rank as gone (regular end of the job: the peers end too)"""
        self._stop.set()

    def wait_for_all(self, timeout_sec: float = 60.0):
        """block until every rank has written its first heartbeat (once, after start-up)"""
        t0 = time.monotonic()
        for r in range(self.world):
            while True:
                try:
                    if self.store.check([self._key(r)]) if hasattr(self.store, "check") else True:
                        self.store.get(self._key(r))
                        break
                except Exception:
                    pass
                if time.monotonic() - t0 > timeout_sec:
                    raise PeerFailure([r], {r: "never sent a heartbeat"})
                time.sleep(0.05)

    def status(self) -> Dict[int, Dict[str, Any]]:
        """state of every rank: ``{"state": "alive" | "left" | "unknown", "step": int, "age": seconds}``"""
        now = self._clock()
        res = {}
        for r in range(self.world):
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    res[r] = {"state": "unknown", "step": -1, "age": float("inf")}
                    continue
                val = self.store.get(self._key(r))
                val = val.decode() if isinstance(val, (bytes, bytearray)) else str(val)
            except Exception as exc:
                res[r] = {"state": "unknown", "step": -1, "age": float("inf"), "error": "%s: %s" % (type(exc).__name__, exc)}
                continue
            if val.startswith("left:"):
                res[r] = {"state": "left", "step": -1, "age": 0.0, "reason": val[5:]}
            else:
                _, step, ts = val.split(":")
                res[r] = {"state": "alive", "step": int(step), "age": max(0.0, now - float(ts))}
        return res

    def failed_ranks(self) -> Dict[int, str]:
        """peers that left or whose heartbeat is stale: rank -> reason"""
        bad = {}
        for r, st in self.status().items():
            if r == self.rank:
                continue
            if st["state"] == "left":
                bad[r] = "left (%s)" % st.get("reason", "")
            elif st["state"] == "unknown":
                bad[r] = "no heartbeat entry"
            elif st["age"] > self.max_age_sec:
                bad[r] = "last heartbeat %.1f s ago at step %i" % (st["age"], st["step"])
        return bad

    def check(self, step: Optional[int] = None):
        """call before issuing a step: raises :class:`PeerFailure` when a peer is gone; records the own step number"""
        if step is not None:
            self._step = int(step)
        bad = self.failed_ranks()
        if bad:
            raise PeerFailure(sorted(bad), bad)


def create_from_process_group(opts: Any, *, rank: int, world: int) -> Optional[PeerWatch]:
    """
    :param opts: the ``peer_watch`` entry of ``torch_distributed``: None / False (off), True (defaults) or a dict
    :return: watch over the default process group's store, after all ranks have reported once
    """
    if not opts or world <= 1:
        return None
    import torch.distributed as dist

    o = dict(opts) if isinstance(opts, dict) else {}
    store = dist.distributed_c10d._get_default_store()
    watch = PeerWatch(store, rank=rank, world=world, interval_sec=float(o.get("interval_sec", 0.5)), max_age_sec=float(o.get("max_age_sec", 10.0)))
    watch.wait_for_all(timeout_sec=float(o.get("startup_timeout_sec", 120.0)))
    return watch
