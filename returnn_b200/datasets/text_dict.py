"""
:class:`TextDictDataset`: a (gzipped) text file holding a Python dict ``{seq_tag: "text"}``; output ``data`` are the labels
from the vocabulary (reference: returnn/datasets/text_dict.py). Large files are parsed by the native literal parser
when the helper library is built.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Union
import gzip
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from .util.vocabulary import Vocabulary


class TextDictDataset(CachedDataset2):
    """tag -> text"""

    def __init__(self, filename: str, vocab: Union[Dict[str, Any], Vocabulary], **kwargs):
        super().__init__(**kwargs)
        from ..utils.literal_py_to_pickle import literal_eval

        raw = (gzip.open(filename, "rb") if filename.endswith(".gz") else open(filename, "rb")).read()
        self._data: Dict[str, str] = literal_eval(raw)
        assert isinstance(self._data, dict)
        self._tags = list(self._data.keys())
        self.vocab = vocab if isinstance(vocab, Vocabulary) else Vocabulary.create_vocab(**vocab)
        self.labels["data"] = list(self.vocab.labels)
        self.num_inputs = self.vocab.num_labels
        self.num_outputs = {"data": (self.vocab.num_labels, 1)}
        self._order: List[int] = []

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            idx = {t: i for i, t in enumerate(self._tags)}
            self._order = [idx[t] for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self._tags), get_seq_len=lambda i: len(self._data[self._tags[i]])))
        self._num_seqs = len(self._order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def get_all_tags(self):
        return list(self._tags)

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._tags)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        tag = self._tags[self._order[seq_idx]]
        return DatasetSeq(seq_idx=seq_idx, seq_tag=tag, features={"data": numpy.array(self.vocab.get_seq(self._data[tag]), dtype="int32")})

    def get_data_dtype(self, key):
        return "int32"

    def is_data_sparse(self, key):
        return True
