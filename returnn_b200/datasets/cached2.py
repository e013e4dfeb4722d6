"""
``CachedDataset2``: base class for streaming datasets. Subclasses implement ``_collect_single_seq(seq_idx)`` returning a
:class:`DatasetSeq` (or None at the end); sequences are requested with increasing index, a small window is kept.

Parity: returnn/datasets/cached2.py:13-130 (CachedDataset2), :269 (SingleStreamPipeDataset).
"""

from __future__ import annotations
from typing import List, Optional, Sequence
import numpy
import threading
from .basic import Dataset, DatasetSeq
from ..utils.basic import NumbersDict

__all__ = ["CachedDataset2", "SingleStreamPipeDataset"]


class CachedDataset2(Dataset):
    """streaming base class"""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self._num_timesteps = None
        self.epoch = None
        self.reached_final_seq = False
        self.added_data: List[DatasetSeq] = []
        self.expected_load_seq_start = 0
        self._num_timesteps_accumulated = NumbersDict(0)

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        """reset the window; subclasses call this first and then set self._num_seqs / their order"""
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if not epoch:
            epoch = 1
        self.expected_load_seq_start = 0
        self.reached_final_seq = False
        self.added_data = []
        self._num_timesteps_accumulated = NumbersDict(0)
        self._num_seqs = None
        self.epoch = epoch
        return True

    def _cleanup_old_seqs(self, seq_idx_end: int):
        i = 0
        while i < len(self.added_data) and self.added_data[i].seq_idx < seq_idx_end:
            i += 1
        del self.added_data[:i]

    def _get_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        for data in self.added_data:
            if data.seq_idx == seq_idx:
                return data
        return None

    def is_cached(self, start, end):
        """always False so that _load_seqs manages the window"""
        return False

    @property
    def num_seqs(self) -> int:
        """known after init_seq_order for most subclasses, else after the end was reached"""
        if self._num_seqs is not None:
            return self._num_seqs
        raise NotImplementedError("%s: num_seqs unknown" % self)

    def _load_seqs(self, start: int, end: int):
        assert start >= self.expected_load_seq_start, "%s: load_seqs must be monotonic (start %i < %i)" % (self, start, self.expected_load_seq_start)
        if start > self.expected_load_seq_start:
            self._cleanup_old_seqs(start)
            self.expected_load_seq_start = start
        if self.added_data:
            start = max(self.added_data[-1].seq_idx + 1, start)
        seqs = []
        for seq_idx in range(start, end):
            seq = self._collect_single_seq(seq_idx)
            if seq is None:
                self.reached_final_seq = True
                if self._num_seqs is None:
                    self._num_seqs = seq_idx
                break
            seqs.append(seq)
        for s in seqs:
            self._num_timesteps_accumulated += s.num_frames
        self.added_data += seqs

    def is_less_than_num_seqs(self, n: int) -> bool:
        """tries to load n when num_seqs is unknown"""
        if n < self.expected_load_seq_start:
            return True
        if self._num_seqs is not None:
            return n < self._num_seqs
        self._load_seqs(self.expected_load_seq_start, n + 1)
        if self._get_seq(n) is not None:
            return True
        return False

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        raise NotImplementedError

    def get_num_timesteps(self):
        """after the end was reached"""
        assert self.reached_final_seq
        return self._num_timesteps_accumulated.get("data", self._num_timesteps_accumulated.max_value() if self._num_timesteps_accumulated.has_values() else 0)

    def get_seq_length(self, seq_idx: int) -> NumbersDict:
        """loads up to seq_idx"""
        if seq_idx >= self.expected_load_seq_start:
            self._load_seqs(self.expected_load_seq_start, seq_idx + 1)
        seq = self._get_seq(seq_idx)
        assert seq is not None, "%s: seq %i not available" % (self, seq_idx)
        return seq.num_frames

    def get_data(self, seq_idx: int, key: str) -> numpy.ndarray:
        seq = self._get_seq(seq_idx)
        assert seq is not None, "%s: seq %i not loaded (window starts at %i)" % (self, seq_idx, self.expected_load_seq_start)
        return seq.features[key]

    def get_input_data(self, seq_idx):
        return self.get_data(seq_idx, "data")

    def get_targets(self, target, seq_idx):
        return self.get_data(seq_idx, target)

    def get_tag(self, sorted_seq_idx: int) -> str:
        seq = self._get_seq(sorted_seq_idx)
        if seq is None and sorted_seq_idx >= self.expected_load_seq_start:
            self._load_seqs(self.expected_load_seq_start, sorted_seq_idx + 1)
            seq = self._get_seq(sorted_seq_idx)
        assert seq is not None
        return seq.seq_tag

    def get_data_keys(self):
        if self.added_data:
            return list(self.added_data[0].features.keys())
        if self.num_outputs:
            keys = list(self.num_outputs.keys())
            if "data" in keys:
                keys.remove("data")
                keys.insert(0, "data")
            return keys
        return super().get_data_keys()

    def get_target_list(self):
        keys = list(self.get_data_keys())
        if "data" in keys:
            keys.remove("data")
        return keys

    def is_data_sparse(self, key):
        if self.added_data and key in self.added_data[0].features:
            arr = self.added_data[0].get_data(key)
            if key in (self.num_outputs or {}):
                return self.num_outputs[key][1] <= 1
            return arr.ndim <= 1 and not str(arr.dtype).startswith("float")
        return super().is_data_sparse(key)

    def get_data_dim(self, key):
        if self.added_data and key not in (self.num_outputs or {}):
            arr = self.added_data[0].get_data(key)
            if arr.ndim >= 2:
                return arr.shape[-1]
        return super().get_data_dim(key)

    def get_data_dtype(self, key):
        if self.added_data and key in self.added_data[0].features:
            return str(self.added_data[0].get_data(key).dtype)
        return super().get_data_dtype(key)


class SingleStreamPipeDataset(CachedDataset2):
    """sequences are pushed in from another thread via ``add(seq)`` / ``finish()``"""

    def __init__(self, dim: int, ndim: int, sparse: bool = False, dtype: str = "float32"):
        super().__init__()
        self.dim, self.ndim, self.sparse, self.dtype = dim, ndim, sparse, dtype
        self.num_inputs = dim
        self.num_outputs = {"data": [dim, ndim]}
        self.is_finished = False
        self.queue: List[numpy.ndarray] = []
        self.condition = threading.Condition()

    def is_data_sparse(self, key):
        return self.sparse

    def get_data_dtype(self, key):
        return self.dtype

    def get_target_list(self):
        return []

    def get_data_keys(self):
        return ["data"]

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        assert not seq_list and not seq_order
        super().init_seq_order(epoch=epoch)
        with self.condition:
            self.is_finished = False
            self.queue[:] = []
        return True

    def finish(self):
        """no more sequences"""
        with self.condition:
            self.is_finished = True
            self.condition.notify_all()

    def add(self, data: numpy.ndarray):
        """push one sequence"""
        with self.condition:
            self.queue.append(data)
            self.condition.notify_all()

    def _collect_single_seq(self, seq_idx):
        with self.condition:
            while True:
                if self.queue:
                    return DatasetSeq(seq_idx=seq_idx, features=self.queue.pop(0))
                if self.is_finished:
                    return None
                self.condition.wait()
