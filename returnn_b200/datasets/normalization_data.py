"""
Mean / standard deviation statistics over a dataset, accumulated in float64 and stored as text or pickle
(reference: returnn/datasets/normalization_data.py).
"""

from __future__ import annotations
from typing import Dict, Optional
import pickle
import numpy


class NormalizationData:
    """running sums per data key"""

    def __init__(self):
        self.sum: Dict[str, numpy.ndarray] = {}
        self.sum_sq: Dict[str, numpy.ndarray] = {}
        self.count: Dict[str, int] = {}

    def update(self, key: str, data: numpy.ndarray):
        """add the frames [T, D] of one sequence"""
        d = numpy.asarray(data, dtype="float64").reshape(data.shape[0], -1)
        if key not in self.sum:
            self.sum[key] = numpy.zeros(d.shape[1])
            self.sum_sq[key] = numpy.zeros(d.shape[1])
            self.count[key] = 0
        self.sum[key] += d.sum(axis=0)
        self.sum_sq[key] += (d * d).sum(axis=0)
        self.count[key] += d.shape[0]

    def mean(self, key: str) -> numpy.ndarray:
        """per-feature mean"""
        return self.sum[key] / max(self.count[key], 1)

    def std_dev(self, key: str) -> numpy.ndarray:
        """per-feature standard deviation"""
        m = self.mean(key)
        return numpy.sqrt(numpy.maximum(self.sum_sq[key] / max(self.count[key], 1) - m * m, 0.0))

    @classmethod
    def from_dataset(cls, dataset, epoch: int = 1, keys=None) -> "NormalizationData":
        """one pass over the dataset"""
        self = cls()
        dataset.init_seq_order(epoch=epoch)
        keys = keys or [k for k in dataset.get_data_keys() if not dataset.is_data_sparse(k) and dataset.get_data_dtype(k).startswith("float")]
        i = 0
        while dataset.is_less_than_num_seqs(i):
            dataset.load_seqs(i, i + 1)
            for k in keys:
                self.update(k, dataset.get_data(i, k))
            i += 1
        return self

    def save(self, filename: str, key: str = "data"):
        """``.pkl``: everything; else text files ``<filename>`` with mean and ``<filename>.std_dev``"""
        if filename.endswith(".pkl"):
            pickle.dump({"sum": self.sum, "sum_sq": self.sum_sq, "count": self.count}, open(filename, "wb"))
            return
        numpy.savetxt(filename, self.mean(key))
        numpy.savetxt(filename + ".std_dev", self.std_dev(key))

    @classmethod
    def load(cls, filename: str) -> "NormalizationData":
        """from ``.pkl``"""
        d = pickle.load(open(filename, "rb"))
        self = cls()
        self.sum, self.sum_sq, self.count = d["sum"], d["sum_sq"], d["count"]
        return self
