"""
Normalisation statistics.

:class:`NormalizationData` holds mean and variance of the inputs and the outputs of a regression corpus, read from a normalisation
HDF file (groups ``inputs`` / ``outputs`` with datasets ``mean``, ``meanOfSquares``, ``variance``, ``totalNumberOfFrames``), and
``create_normalization_file`` computes such a file over all HDF files of a bundle (reference: returnn/datasets/normalization_data.py).
The same class also accumulates running sums over any dataset (``update`` / ``from_dataset`` / ``save`` / ``load``), which the
statistics tools use.
"""

from __future__ import annotations
from typing import Dict, Optional
import pickle
import numpy


class NormalizationData:
    """running sums per data key"""

    GROUP_INPUTS, GROUP_OUTPUTS = "inputs", "outputs"
    DATASET_MEAN, DATASET_MEAN_OF_SQUARES, DATASET_VARIANCE, DATASET_TOTAL_FRAMES = "mean", "meanOfSquares", "variance", "totalNumberOfFrames"

    def __init__(self, normalizationFilePath: Optional[str] = None):
        """:param normalizationFilePath: a normalisation HDF file to read (None: empty, for accumulation)"""
        self._input_mean = self._input_variance = self._output_mean = self._output_variance = None
        if normalizationFilePath is not None:
            from ..utils.h5_shim import get_h5py

            with get_h5py().File(normalizationFilePath, "r") as f:
                self._input_mean, self._input_variance = self._getMeanAndVarianceFromGroup(f, self.GROUP_INPUTS)
                self._output_mean, self._output_variance = self._getMeanAndVarianceFromGroup(f, self.GROUP_OUTPUTS)
        self.sum: Dict[str, numpy.ndarray] = {}
        self.sum_sq: Dict[str, numpy.ndarray] = {}
        self.count: Dict[str, int] = {}

    @classmethod
    def _getMeanAndVarianceFromGroup(cls, f, group_name: str):
        if group_name not in f:
            return None, None
        g = f[group_name]
        mean = numpy.asarray(g[cls.DATASET_MEAN][...]) if cls.DATASET_MEAN in g else None
        var = numpy.asarray(g[cls.DATASET_VARIANCE][...]) if cls.DATASET_VARIANCE in g else None
        return mean, var

    @property
    def inputMean(self):
        """mean of the inputs ``[features]`` or None"""
        return self._input_mean

    @property
    def inputVariance(self):
        """variance of the inputs or None"""
        return self._input_variance

    @property
    def outputMean(self):
        """mean of the outputs or None"""
        return self._output_mean

    @property
    def outputVariance(self):
        """variance of the outputs or None"""
        return self._output_variance

    @classmethod
    def create_normalization_file(cls, bundle_file_path: str, output_file_path: str, dtype=numpy.float64, flag_include_outputs: bool = True):
        """
        Statistics over the ``inputs`` (and ``outputs``) groups of all HDF files listed in the bundle file, written to
        ``output_file_path`` in the layout described in the module docstring.
        """
        from ..utils.h5_shim import get_h5py
        from .bundle_file import BundleFile

        h5py = get_h5py()
        groups = [cls.GROUP_INPUTS] + ([cls.GROUP_OUTPUTS] if flag_include_outputs else [])
        with h5py.File(output_file_path, "w") as out:
            for group_name in groups:
                total = total_sq = None
                frames = 0
                for path in BundleFile(bundle_file_path).dataset_file_paths:
                    with h5py.File(path, "r") as f:
                        if group_name not in f:
                            continue
                        for name in f[group_name].keys():
                            d = numpy.asarray(f[group_name][name][...], dtype=dtype)
                            total = d.sum(axis=0) if total is None else total + d.sum(axis=0)
                            total_sq = (d * d).sum(axis=0) if total_sq is None else total_sq + (d * d).sum(axis=0)
                            frames += d.shape[0]
                if total is None:
                    continue
                mean = total / frames
                mean_sq = total_sq / frames
                g = out.create_group(group_name)
                g.create_dataset(cls.DATASET_MEAN, data=mean.astype(dtype))
                g.create_dataset(cls.DATASET_MEAN_OF_SQUARES, data=mean_sq.astype(dtype))
                g.create_dataset(cls.DATASET_VARIANCE, data=numpy.maximum(mean_sq - mean * mean, 0.0).astype(dtype))
                g.create_dataset(cls.DATASET_TOTAL_FRAMES, data=numpy.array(frames))

    createNormalizationFile = create_normalization_file

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
