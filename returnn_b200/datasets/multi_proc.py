"""
:class:`MultiProcDataset`: N worker processes each hold a copy of the wrapped dataset and load every N-th sequence
of the epoch order; the parent reads them round-robin, so the result is deterministic and identical to the wrapped
dataset read in one process (reference: returnn/datasets/multi_proc.py:22-510).

The sequence order is computed once per epoch in the parent (``seq_order`` is then sent to the workers), workers
prefetch up to ``buffer_size`` sequences each. Workers are spawned with the non-daemonic spawn context so that they may
have children of their own.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Union
import sys
import numpy
from .basic import Dataset, DatasetSeq, init_dataset
from .cached2 import CachedDataset2
from ..utils.multi_proc_non_daemonic_spawn import NonDaemonicSpawnContext

_mp = NonDaemonicSpawnContext(process_pre_init_func=None)


def _worker_main(conn, dataset_opts: Dict[str, Any], worker_idx: int, num_workers: int, buffer_size: int):
    """child process: serve ``init`` / ``get`` / ``exit`` messages"""
    try:
        ds = init_dataset(dataset_opts)
        order: List[int] = []
        pos = 0
        while True:
            msg, arg = conn.recv()
            if msg == "exit":
                break
            if msg == "init":
                epoch, seq_order, seq_list = arg
                if seq_order is not None:
                    mine = list(seq_order)[worker_idx::num_workers]
                    ds.init_seq_order(epoch=epoch, seq_order=mine)
                elif seq_list is not None:
                    ds.init_seq_order(epoch=epoch, seq_list=list(seq_list)[worker_idx::num_workers])
                else:
                    raise ValueError("worker needs an explicit order")
                pos = 0
                conn.send(("ok", None))
            elif msg == "get":
                n = arg
                out = []
                for _ in range(n):
                    if not ds.is_less_than_num_seqs(pos):
                        out.append(None)
                        break
                    ds.load_seqs(pos, pos + 1)
                    out.append((ds.get_tag(pos), {k: ds.get_data(pos, k) for k in ds.get_data_keys()}))
                    pos += 1
                conn.send(("seqs", out))
            elif msg == "meta":
                conn.send(("meta", {"keys": ds.get_data_keys(), "targets": ds.get_target_list(), "num_outputs": ds.num_outputs,
                                    "num_inputs": ds.num_inputs, "labels": ds.labels,
                                    "dtypes": {k: ds.get_data_dtype(k) for k in ds.get_data_keys()},
                                    "total": ds.get_total_num_seqs() if _can(ds.get_total_num_seqs) else None,
                                    "tags": ds.get_all_tags() if _can(ds.get_all_tags) else None}))
    except KeyboardInterrupt:
        pass
    except Exception as exc:  # report to the parent instead of dying silently
        try:
            conn.send(("error", "%s: %s" % (type(exc).__name__, exc)))
        except Exception:
            pass
        raise


def _can(fn) -> bool:
    try:
        fn()
        return True
    except Exception:
        return False


class MultiProcDataset(CachedDataset2):
    """wrapped dataset loaded by worker processes"""

    def __init__(self, dataset: Dict[str, Any], num_workers: int, buffer_size: int, sharding_method: str = "seq_order", **kwargs):
        super().__init__(**kwargs)
        assert num_workers > 0 and buffer_size > 0
        assert sharding_method in ("seq_order", "dedicated")
        self.dataset_opts = dataset
        self.num_workers = num_workers
        self.buffer_size = buffer_size
        self.sharding_method = sharding_method
        self._procs = None
        self._conns = None
        self._order_ds: Optional[Dataset] = None
        self._meta = None
        self._buffers: List[List] = []
        self._finished: List[bool] = []
        self._lazy_init()

    def _lazy_init(self):
        if self._procs is not None:
            return
        self._procs, self._conns = [], []
        for i in range(self.num_workers):
            parent, child = _mp.Pipe()
            p = _mp.Process(target=_worker_main, args=(child, self.dataset_opts, i, self.num_workers, self.buffer_size), daemon=True,
                            name="%s worker %i" % (self.name, i))
            p.start()
            child.close()
            self._procs.append(p)
            self._conns.append(parent)
        self._conns[0].send(("meta", None))
        kind, meta = self._recv(0)
        assert kind == "meta"
        self._meta = meta
        self.num_outputs, self.num_inputs, self.labels = meta["num_outputs"], meta["num_inputs"], meta["labels"] or {}
        # the parent keeps a copy only to compute the epoch order (never loads data from it)
        self._order_ds = init_dataset(self.dataset_opts)

    def _recv(self, i: int):
        kind, payload = self._conns[i].recv()
        if kind == "error":
            raise RuntimeError("%s: worker %i failed: %s" % (self, i, payload))
        return kind, payload

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        self._lazy_init()
        if seq_order is None and seq_list is None:
            self._order_ds.init_seq_order(epoch=epoch)
            seq_order = list(self._order_ds.get_current_seq_order())
        total = len(seq_order) if seq_order is not None else len(seq_list)
        for c in self._conns:
            c.send(("init", (epoch, seq_order, seq_list)))
        for i in range(self.num_workers):
            self._recv(i)
        self._buffers = [[] for _ in range(self.num_workers)]
        self._finished = [False] * self.num_workers
        self._num_seqs = total
        return True

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= self._num_seqs:
            return None
        w = seq_idx % self.num_workers
        if not self._buffers[w] and not self._finished[w]:
            self._conns[w].send(("get", self.buffer_size))
            _, seqs = self._recv(w)
            for s in seqs:
                if s is None:
                    self._finished[w] = True
                else:
                    self._buffers[w].append(s)
        if not self._buffers[w]:
            return None
        tag, feats = self._buffers[w].pop(0)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=tag, features=feats)

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        if self._meta["total"] is None:
            raise NotImplementedError
        return self._meta["total"]

    def get_all_tags(self):
        if self._meta["tags"] is None:
            raise NotImplementedError
        return list(self._meta["tags"])

    def get_data_keys(self):
        return list(self._meta["keys"])

    def get_target_list(self):
        return list(self._meta["targets"])

    def get_data_dtype(self, key):
        return self._meta["dtypes"][key]

    def get_data_dim(self, key):
        return self.num_outputs[key][0]

    def is_data_sparse(self, key):
        return self.num_outputs[key][1] == 1

    def get_data_shape(self, key):
        return [] if self.is_data_sparse(key) else [self.num_outputs[key][0]]

    def finish_epoch(self, *, free_resources: bool = False):
        super().finish_epoch(free_resources=free_resources)
        if free_resources:
            self._exit_workers()

    def _exit_workers(self):
        if not self._procs:
            return
        for c in self._conns:
            try:
                c.send(("exit", None))
            except Exception:
                pass
        for p in self._procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
        self._procs = None
        self._conns = None

    def __del__(self):
        try:
            self._exit_workers()
        except Exception:
            pass

    def __getstate__(self):
        d = dict(self.__dict__)
        d["_procs"] = d["_conns"] = d["_order_ds"] = None
        return d
