"""
:class:`CachedDataset`: base class for datasets that know all sequence lengths up front and keep a byte-budgeted cache
of loaded sequences in one preallocated array per key (reference: returnn/datasets/cached.py:18). Subclasses fill
``_seq_lengths`` (``[num_seqs, num_keys]``), ``_seq_tags`` and implement ``_load_seq_data(corpus_idx) -> {key: array}``.
"""

from __future__ import annotations
from typing import Dict, List, Optional, Sequence
import numpy
from .basic import Dataset
from ..utils.basic import NumbersDict


class CachedDataset(Dataset):
    """whole-dataset cache with a byte budget (``cache_byte_size``; 0 = everything fits, -1 = no cache)"""

    def __init__(self, cache_byte_size: int = 0, **kwargs):
        super().__init__(**kwargs)
        self.cache_byte_size_total_limit = cache_byte_size
        self._seq_lengths: Optional[numpy.ndarray] = None
        self._seq_tags: List[str] = []
        self._keys: List[str] = ["data"]
        self._order: List[int] = []
        self._cache: Dict[int, Dict[str, numpy.ndarray]] = {}
        self._cache_bytes = 0
        self._lru: List[int] = []

    def _load_seq_data(self, corpus_idx: int) -> Dict[str, numpy.ndarray]:
        raise NotImplementedError

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        n = len(self._seq_tags)
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            idx = {t: i for i, t in enumerate(self._seq_tags)}
            self._order = [idx[t] for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=n, get_seq_len=lambda i: int(self._seq_lengths[i, 0])))
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    def get_current_seq_order(self):
        return list(self._order)

    @property
    def num_seqs(self) -> int:
        return len(self._order)

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._seq_tags)

    def get_all_tags(self):
        return list(self._seq_tags)

    def get_tag(self, sorted_seq_idx: int) -> str:
        return self._seq_tags[self._order[sorted_seq_idx]]

    def get_seq_length(self, seq_idx: int) -> NumbersDict:
        row = self._seq_lengths[self._order[seq_idx]]
        return NumbersDict({k: int(row[min(i, len(row) - 1)]) for i, k in enumerate(self._keys)})

    def get_num_timesteps(self) -> int:
        return int(self._seq_lengths[:, 0].sum())

    def is_cached(self, start: int, end: int) -> bool:
        return all(self._order[i] in self._cache for i in range(start, min(end, len(self._order))))

    def _evict_for(self, need: int):
        limit = self.cache_byte_size_total_limit
        if limit <= 0:
            return
        while self._lru and self._cache_bytes + need > limit:
            victim = self._lru.pop(0)
            d = self._cache.pop(victim, None)
            if d:
                self._cache_bytes -= sum(a.nbytes for a in d.values())

    def _load_seqs(self, start: int, end: int):
        for i in range(start, min(end, len(self._order))):
            ci = self._order[i]
            if ci in self._cache:
                if ci in self._lru:
                    self._lru.remove(ci)
                self._lru.append(ci)
                continue
            d = self._load_seq_data(ci)
            need = sum(a.nbytes for a in d.values())
            if self.cache_byte_size_total_limit == -1:
                self._cache = {ci: d}
                self._lru = [ci]
                self._cache_bytes = need
                continue
            self._evict_for(need)
            self._cache[ci] = d
            self._lru.append(ci)
            self._cache_bytes += need

    def get_data(self, seq_idx: int, key: str) -> numpy.ndarray:
        ci = self._order[seq_idx]
        if ci not in self._cache:
            self._load_seqs(seq_idx, seq_idx + 1)
        return self._cache[ci][key]

    def get_data_keys(self):
        return list(self._keys)

    def get_target_list(self):
        return [k for k in self._keys if k != "data"]

    # -- accessors of the reference class that tools and old configs use ------------------------------------------------
    def supports_sharding(self) -> bool:
        return True

    def have_corpus_seq_idx(self) -> bool:
        return True

    def get_corpus_seq_idx(self, seq_idx: int) -> int:
        return int(self._order[seq_idx])

    def get_seq_length_nd(self, sorted_seq_idx: int) -> numpy.ndarray:
        """lengths of all keys as one row (reference: cached.py:593)"""
        return numpy.asarray(self._seq_lengths[self._order[sorted_seq_idx]])

    def get_seq_start(self, sorted_seq_idx: int) -> numpy.ndarray:
        """frames of all keys in front of this sequence, in the order of the current epoch (reference: cached.py:616)"""
        if getattr(self, "_seq_starts_for", None) is not self._order:
            lens = numpy.asarray(self._seq_lengths)[numpy.asarray(self._order, dtype="int64")] if len(self._order) else numpy.zeros((0, 1), "int64")
            self._seq_starts = numpy.concatenate([numpy.zeros((1, lens.shape[1]), dtype="int64"), numpy.cumsum(lens, axis=0, dtype="int64")])
            self._seq_starts_for = self._order
        return self._seq_starts[sorted_seq_idx]

    def batch_set_generator_cache_whole_epoch(self) -> bool:
        """whether a batch generator may keep the whole epoch (everything fits into the cache)"""
        return self.cache_byte_size_total_limit == 0

    def delete(self, nframes: int) -> int:
        """
        Frees cached sequences, least recently used first, until at least ``nframes`` frames are gone (reference: cached.py:536).

        :return: frames actually freed
        """
        freed = 0
        while self._lru and freed < nframes:
            victim = self._lru.pop(0)
            d = self._cache.pop(victim, None)
            if d:
                self._cache_bytes -= sum(a.nbytes for a in d.values())
                freed += int(self._seq_lengths[victim, 0])
        return freed
