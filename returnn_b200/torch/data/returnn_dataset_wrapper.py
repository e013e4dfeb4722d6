"""
Wrap a :class:`returnn_b200.datasets.Dataset` as a ``torch.utils.data.IterableDataset`` that yields one dict per
sequence: all data keys plus ``seq_tag``, ``seq_idx``, ``epoch``, ``num_seqs``, ``complete_frac``.

The epoch is handed over through a multiprocessing-shared integer so that DataLoader worker processes (which hold a
pickled copy of the dataset) re-initialise their sequence order for every new epoch.

Parity: returnn/torch/data/returnn_dataset_wrapper.py:46-149.
"""

from __future__ import annotations
from typing import Callable, Dict, Iterable, Optional
import numpy
import torch.utils.data
from ...datasets.basic import Dataset

ResetCallbackT = Callable[[], None]


class ReturnnDatasetResetDefaultEpochCounterCallback:
    """counts epochs locally (used when nobody provides the epoch from outside)"""

    def __init__(self, dataset: Dataset):
        self.dataset = dataset
        self.epoch = 0

    def __call__(self):
        self.epoch += 1
        self.dataset.init_seq_order(epoch=self.epoch)


class ReturnnDatasetResetMpSharedEpochCallback:
    """reads the epoch from a multiprocessing-shared value written by the engine"""

    def __init__(self, dataset: Dataset, epoch_mp_shared):
        self.dataset = dataset
        self.epoch_mp_shared = epoch_mp_shared

    def __call__(self):
        epoch = self.epoch_mp_shared.value
        self.dataset.init_seq_order(epoch=epoch or None)


class ReturnnDatasetResetNoOpCallback:
    """the caller initialised the order already"""

    def __call__(self):
        pass


class ReturnnDatasetIterDataPipe(torch.utils.data.IterableDataset):
    """iterates the dataset sequence by sequence"""

    def __init__(self, returnn_dataset: Dataset, *, reset_callback: Optional[ResetCallbackT] = None):
        super().__init__()
        self._dataset = returnn_dataset
        if not reset_callback:
            reset_callback = ReturnnDatasetResetDefaultEpochCounterCallback(returnn_dataset)
        self._reset_callback = reset_callback

    def reset(self):
        """new epoch"""
        self._reset_callback()

    def __iter__(self) -> Iterable[Dict[str, numpy.ndarray]]:
        self.reset()
        ds = self._dataset
        try:
            num_seqs = ds.num_seqs
            if num_seqs == float("inf"):
                num_seqs = -1
        except Exception:
            num_seqs = -1
        num_seqs = numpy.array(num_seqs, dtype="int64")
        epoch = numpy.array(ds.epoch or 1, dtype="int32")
        keys = ds.get_data_keys()
        seq_index = 0
        while ds.is_less_than_num_seqs(seq_index):
            ds.load_seqs(seq_index, seq_index + 1)
            data = {k: ds.get_data(seq_index, k) for k in keys}
            data["seq_tag"] = numpy.array(ds.get_tag(seq_index))
            data["seq_idx"] = numpy.array(seq_index, dtype="int64")
            data["epoch"] = epoch
            data["num_seqs"] = num_seqs
            frac = ds.get_complete_frac(seq_index, allow_only_lr_suitable=True)
            data["complete_frac"] = numpy.array(-1.0 if frac is None else frac, dtype="float32")
            yield data
            seq_index += 1

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


class ReturnnDatasetPerEpochMapDataPipe(torch.utils.data.Dataset):
    """map-style access for datasets with random access (``have_get_corpus_seq``)"""

    def __init__(self, returnn_dataset: Dataset, *, reset_callback: Optional[ResetCallbackT] = None):
        super().__init__()
        assert returnn_dataset.have_corpus_seq_idx() and returnn_dataset.have_get_corpus_seq()
        self._dataset = returnn_dataset
        if not reset_callback:
            reset_callback = ReturnnDatasetResetDefaultEpochCounterCallback(returnn_dataset)
        self._reset_callback = reset_callback

    def reset(self):
        """new epoch"""
        self._reset_callback()

    def __len__(self):
        return self._dataset.num_seqs

    def __getitem__(self, index):
        corpus_seq_idx = self._dataset.get_corpus_seq_idx(index)
        seq = self._dataset.get_corpus_seq(corpus_seq_idx)
        return seq.features


class ReturnnDatasetFullMapDataPipe(torch.utils.data.Dataset):
    """
    Map-style view of a whole dataset in its corpus order (``dataset.have_get_corpus_seq()`` must hold): index -> ``{key: array}``.
    Ordering and shuffling are left to the torch side of the pipeline. Parity: returnn/torch/data/returnn_dataset_wrapper.py:194.
    """

    def __init__(self, returnn_dataset):
        assert returnn_dataset.have_get_corpus_seq(), "%r cannot be read by corpus index" % returnn_dataset
        self._dataset = returnn_dataset

    def __len__(self) -> int:
        return self._dataset.get_total_num_seqs()

    def __getitem__(self, index: int):
        return self._dataset.get_corpus_seq(index).features
