"""
:class:`NumpyDumpDataset`: a directory of ``<prefix><idx><postfix_data>`` / ``...<postfix_targets>`` text dumps written
with ``numpy.savetxt`` (reference: returnn/datasets/numpy_dump.py).
"""

from __future__ import annotations
from typing import List, Optional
import os
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2


class NumpyDumpDataset(CachedDataset2):
    """one pair of text files per sequence"""

    file_format_data = "%i.data"
    file_format_targets = "%i.targets"

    def __init__(self, prefix: str, postfix: str = ".txt.gz", start_seq: int = 0, end_seq: Optional[int] = None, num_inputs: Optional[int] = None,
                 num_outputs=None, **kwargs):
        super().__init__(**kwargs)
        self.file_format_data = prefix + self.file_format_data + postfix
        self.file_format_targets = prefix + self.file_format_targets + postfix
        self.start_seq = start_seq
        if end_seq is None:
            end_seq = start_seq
            while os.path.exists(self.file_format_data % end_seq):
                end_seq += 1
        self.end_seq = end_seq
        assert num_inputs and num_outputs
        self.num_inputs = num_inputs
        self.num_outputs = num_outputs if isinstance(num_outputs, dict) else {"data": (num_inputs, 2), "classes": (num_outputs, 1)}
        self._order: List[int] = []

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        n = self.end_seq - self.start_seq
        self._order = list(seq_order) if seq_order is not None else list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=n))
        self._num_seqs = len(self._order)
        return True

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        real = self._order[seq_idx] + self.start_seq
        data = numpy.loadtxt(self.file_format_data % real).astype("float32")
        if data.ndim == 1:
            data = data[:, None]
        targets = numpy.loadtxt(self.file_format_targets % real).astype("int32").reshape(-1)
        return DatasetSeq(seq_idx=seq_idx, seq_tag="seq-%i" % real, features=data, targets={"classes": targets})
