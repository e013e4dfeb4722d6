"""
Regression ("stereo") datasets: parallel input and output feature sequences, e.g. noisy and clean speech features.

:class:`StereoHdfDataset` reads HDF files with a group ``inputs`` and, for training, a group ``outputs``, each holding one 2-D
dataset ``[time, features]`` per sequence named ``"0"``, ``"1"``, ...  Several files can be given through a ``.bundle`` file
(:class:`~returnn_b200.datasets.bundle_file.BundleFile`). Optional mean / variance normalisation from a normalisation file
(:class:`~returnn_b200.datasets.normalization_data.NormalizationData`). :class:`DatasetWithTimeContext` stacks ``tau`` neighbouring
frames on both sides of every input frame.  Reference: returnn/datasets/stereo.py:21-451.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Tuple
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from .bundle_file import BundleFile


class StereoDataset(CachedDataset2):
    """
    Base of the regression datasets: the subclass says how many sequences there are (``_get_total_number_of_sequences``) and reads
    one (``_collect_single_seq``); this class does ordering and epoch partitioning.
    """

    def __init__(self, partition_epoch: int = 1, **kwargs):
        super().__init__(partition_epoch=partition_epoch, **kwargs)
        self._seq_index_list: Optional[List[int]] = None

    def initialize(self):
        self._num_seqs = self._get_total_number_of_sequences()
        super().initialize()

    def _get_total_number_of_sequences(self) -> int:
        raise NotImplementedError

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return self._get_total_number_of_sequences()

    @property
    def num_seqs(self) -> int:
        return len(self._seq_index_list) if self._seq_index_list is not None else self._get_total_number_of_sequences()

    @property
    def seqs_per_epoch(self) -> int:
        """sequences in one (sub)epoch"""
        return self.num_seqs

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._seq_index_list = list(seq_order)
        elif seq_list is not None:
            self._seq_index_list = [int(t.split("-")[-1]) for t in seq_list]
        else:
            self._seq_index_list = list(self.get_seq_order_for_epoch(epoch or 1, self._get_total_number_of_sequences(), lambda i: self._seq_len(i)))
        self._num_seqs = len(self._seq_index_list)
        return True

    def _seq_len(self, corpus_idx: int) -> int:
        return 1

    def get_current_seq_order(self):
        return list(self._seq_index_list or [])

    def supports_seq_order_sorting(self) -> bool:
        return True


class StereoHdfDataset(StereoDataset):
    """inputs (and outputs) from HDF files, see the module docstring"""

    def __init__(self, hdfFile: str, num_outputs: Optional[int] = None, normalizationFile: Optional[str] = None,
                 flag_normalizeInputs: bool = True, flag_normalizeTargets: bool = True, **kwargs):
        super().__init__(**kwargs)
        from ..utils.h5_shim import get_h5py

        h5py = get_h5py()
        paths = BundleFile(hdfFile).dataset_file_paths if hdfFile.endswith(".bundle") else [hdfFile]
        self._files = [h5py.File(p, "r") for p in paths]
        self._seq_map: List[Tuple[int, str]] = []  # corpus seq idx -> (file idx, dataset name)
        for fi, f in enumerate(self._files):
            names = sorted(f["inputs"].keys(), key=lambda s: int(s))
            self._seq_map.extend((fi, n) for n in names)
        self._has_outputs = all("outputs" in f for f in self._files)
        self._norm = None
        self._norm_inputs, self._norm_targets = flag_normalizeInputs, flag_normalizeTargets
        if normalizationFile is not None:
            from .normalization_data import NormalizationData

            self._norm = NormalizationData(normalizationFile)
        first = self._files[0]["inputs"][self._seq_map[0][1]]
        self.num_inputs = int(first.shape[1])
        if self._has_outputs:
            out_dim = int(self._files[0]["outputs"][self._seq_map[0][1]].shape[1])
        else:
            if num_outputs is None:
                raise ValueError("StereoHdfDataset: the file has no 'outputs' group, so num_outputs must be given")
            out_dim = int(num_outputs)
        self.num_outputs = {"data": (self.num_inputs, 2), "classes": (out_dim, 2)}

    def _get_total_number_of_sequences(self) -> int:
        return len(self._seq_map)

    def _seq_len(self, corpus_idx: int) -> int:
        fi, name = self._seq_map[corpus_idx]
        return int(self._files[fi]["inputs"][name].shape[0])

    def get_data_dim(self, key: str) -> int:
        return self.num_outputs[key][0]

    def get_data_dtype(self, key: str) -> str:
        return "float32"

    def is_data_sparse(self, key: str) -> bool:
        return False

    @staticmethod
    def _normalizeVector(v: numpy.ndarray, mean: numpy.ndarray, variance: numpy.ndarray) -> numpy.ndarray:
        return (v - mean) / numpy.sqrt(variance)

    def _read(self, corpus_idx: int) -> Tuple[numpy.ndarray, Optional[numpy.ndarray]]:
        fi, name = self._seq_map[corpus_idx]
        x = numpy.asarray(self._files[fi]["inputs"][name][...], dtype="float32")
        y = numpy.asarray(self._files[fi]["outputs"][name][...], dtype="float32") if self._has_outputs else None
        if self._norm is not None:
            if self._norm_inputs and self._norm.inputMean is not None:
                x = self._normalizeVector(x, self._norm.inputMean, self._norm.inputVariance).astype("float32")
            if y is not None and self._norm_targets and self._norm.outputMean is not None:
                y = self._normalizeVector(y, self._norm.outputMean, self._norm.outputVariance).astype("float32")
        return x, y

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if self._seq_index_list is None or seq_idx >= len(self._seq_index_list):
            return None
        corpus_idx = self._seq_index_list[seq_idx]
        x, y = self._read(corpus_idx)
        return DatasetSeq(seq_idx=seq_idx, seq_tag="seq-%i" % corpus_idx, features=x, targets=y)

    def get_data_keys(self):
        return ["data", "classes"] if self._has_outputs else ["data"]

    def get_target_list(self):
        return ["classes"] if self._has_outputs else []


class DatasetWithTimeContext(StereoHdfDataset):
    """input frame t becomes ``[x[t - tau], ..., x[t], ..., x[t + tau]]`` (edges padded by repeating the first / last frame)"""

    def __init__(self, hdfFile: str, tau: int = 1, **kwargs):
        if tau <= 0:
            raise ValueError("DatasetWithTimeContext: tau must be greater than zero")
        super().__init__(hdfFile, **kwargs)
        self._tau = tau
        self.num_inputs = self.num_inputs * (2 * tau + 1)
        self.num_outputs["data"] = (self.num_inputs, 2)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        seq = super()._collect_single_seq(seq_idx)
        if seq is None:
            return None
        x = seq.features["data"]
        t = x.shape[0]
        idx = numpy.clip(numpy.arange(t)[:, None] + numpy.arange(-self._tau, self._tau + 1)[None, :], 0, t - 1)
        seq.features["data"] = x[idx].reshape(t, -1)
        return seq
