"""
Map-style datasets: subclass :class:`MapDatasetBase` (``__len__``, ``__getitem__`` returning ``{key: numpy array}``) and
wrap it with :class:`MapDatasetWrapper` to get the full Dataset API (reference: returnn/datasets/map.py).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2


class MapDatasetBase:
    """random-access container of sequences"""

    def __init__(self, data_types: Optional[Dict[str, Dict[str, Any]]] = None):
        self.data_types = data_types or {}

    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, seq_idx: int) -> Dict[str, numpy.ndarray]:
        raise NotImplementedError

    def get_seq_len(self, seq_idx: int) -> Optional[int]:
        """length for sorting, None if not known without loading"""
        return None

    def get_seq_tag(self, seq_idx: int) -> str:
        """tag"""
        return "seq-%i" % seq_idx

    def get_seq_order(self, epoch: Optional[int] = None) -> Optional[Sequence[int]]:
        """custom order, or None to use seq_ordering of the wrapper"""
        return None


class FromListDataset(MapDatasetBase):
    """list of dicts"""

    def __init__(self, data_list: List[Dict[str, numpy.ndarray]], sort_data_key: Optional[str] = None, **kwargs):
        super().__init__(**kwargs)
        self._data = data_list
        self._sort_key = sort_data_key

    def __len__(self):
        return len(self._data)

    def __getitem__(self, i):
        return self._data[i]

    def get_seq_len(self, i):
        return len(self._data[i][self._sort_key]) if self._sort_key else None


class MapDatasetWrapper(CachedDataset2):
    """Dataset API over a MapDatasetBase"""

    def __init__(self, map_dataset, **kwargs):
        super().__init__(**kwargs)
        if callable(map_dataset) and not isinstance(map_dataset, MapDatasetBase):
            map_dataset = map_dataset(**{})
        self._ds: MapDatasetBase = map_dataset
        self._order: List[int] = []
        self.num_outputs = {}
        for key, opts in self._ds.data_types.items():
            shape = opts.get("shape", (None, opts.get("dim")))
            sparse = opts.get("sparse", False)
            self.num_outputs[key] = (opts.get("dim") or (shape[-1] if shape else 1), len(shape) if not sparse else len(shape))
        self.num_inputs = self.num_outputs.get("data", (0, 0))[0]

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            idx = {self._ds.get_seq_tag(i): i for i in range(len(self._ds))}
            self._order = [idx[t] for t in seq_list]
        else:
            custom = self._ds.get_seq_order(epoch=epoch)
            if custom is not None:
                self._order = list(custom)
            else:
                have_len = len(self._ds) > 0 and self._ds.get_seq_len(0) is not None
                self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self._ds), get_seq_len=self._ds.get_seq_len if have_len else None))
        self._num_seqs = len(self._order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return len(self._ds) > 0 and self._ds.get_seq_len(0) is not None

    def get_current_seq_order(self):
        return list(self._order)

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._ds)

    def get_all_tags(self):
        return [self._ds.get_seq_tag(i) for i in range(len(self._ds))]

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        ci = self._order[seq_idx]
        d = self._ds[ci]
        tag = d.pop("seq_tag") if "seq_tag" in d else self._ds.get_seq_tag(ci)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=str(tag), features={k: numpy.asarray(v) for k, v in d.items()})

    def get_data_keys(self):
        return list(self._ds.data_types.keys()) or ["data"]

    def get_target_list(self):
        return [k for k in self.get_data_keys() if k != "data"]

    def get_data_dtype(self, key):
        return self._ds.data_types.get(key, {}).get("dtype", "float32")

    def is_data_sparse(self, key):
        return bool(self._ds.data_types.get(key, {}).get("sparse", False))

    def get_data_dim(self, key):
        return self.num_outputs[key][0]

    def get_data_shape(self, key):
        shape = list(self._ds.data_types.get(key, {}).get("shape", (None,)))
        return shape[1:]
