"""
HDF5 datasets and writers (reference: returnn/datasets/hdf.py).

File layout of :class:`HDFDataset` (written by :class:`SimpleHDFWriter` / :class:`HDFDatasetWriter`):
``inputs`` ``[total_frames, dim]`` (or ``[total_frames]`` when sparse), ``seqLengths`` ``[num_seqs, 1 + num_targets]``,
``seqTags`` ``[num_seqs]``, ``targets/data/<key>``, ``targets/size/<key>`` (attrs: dim, ndim), ``targets/labels/<key>``,
file attrs ``inputPattSize``, ``numSeqs``, ``numTimesteps``, ``numLabels``.

``h5py`` is an optional dependency: the classes import it on first use and raise an error that names the package when
it is missing. ``NpzDataset`` / ``NpzWriter`` below keep the same logical layout in a ``.npz`` file for environments
without HDF5.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Union
import os
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from ..utils.basic import NumbersDict


def _h5py():
    try:
        import h5py
    except ImportError as exc:
        raise ImportError("HDFDataset / SimpleHDFWriter need the h5py package, which is not installed here: %s "
                          "(NpzDataset / NpzWriter keep the same layout without HDF5)" % exc)
    return h5py


class _Layout:
    """the logical content of one file, independent of the container format"""

    def __init__(self):
        self.inputs: Optional[numpy.ndarray] = None
        self.seq_lengths: Optional[numpy.ndarray] = None  # [num_seqs, 1 + num_targets]
        self.seq_tags: List[str] = []
        self.targets: Dict[str, numpy.ndarray] = {}
        self.target_dims: Dict[str, tuple] = {}  # key -> (dim, ndim)
        self.labels: Dict[str, List[str]] = {}
        self.input_dim = 0
        self.input_ndim = 2
        self.target_keys: List[str] = []


class HDFDataset(CachedDataset2):
    """reads one or several files of the layout above; sequences are numbered over all files"""

    def __init__(self, files: Optional[Sequence[str]] = None, use_cache_manager: bool = False, **kwargs):
        super().__init__(**kwargs)
        self.files: List[str] = []
        self._layouts: List[_Layout] = []
        self._file_seq_start: List[int] = [0]
        self._seq_starts: List[numpy.ndarray] = []
        self._order: List[int] = []
        self.num_outputs = {}
        self.num_inputs = 0
        for fn in files or []:
            self.add_file(fn)

    def _read(self, filename: str) -> _Layout:
        h5py = _h5py()
        lay = _Layout()
        with h5py.File(filename, "r") as f:
            lay.inputs = f["inputs"][...]
            lay.seq_lengths = f["seqLengths"][...]
            if lay.seq_lengths.ndim == 1:
                lay.seq_lengths = lay.seq_lengths[:, None]
            lay.seq_tags = [t.decode("utf8") if isinstance(t, bytes) else str(t) for t in f["seqTags"][...]]
            if "targets" in f:
                for key in f["targets/data"]:
                    lay.targets[key] = f["targets/data"][key][...]
                    size = f["targets/size"].attrs[key]
                    lay.target_dims[key] = (int(size[0]), int(size[1])) if numpy.ndim(size) else (int(size), 1)
                    if "labels" in f["targets"] and key in f["targets/labels"]:
                        lay.labels[key] = [x.decode("utf8") if isinstance(x, bytes) else str(x) for x in f["targets/labels"][key][...]]
                lay.target_keys = sorted(lay.targets.keys())
            lay.input_ndim = lay.inputs.ndim
            lay.input_dim = int(f.attrs.get("inputPattSize", lay.inputs.shape[1] if lay.inputs.ndim > 1 else int(lay.inputs.max()) + 1))
        return lay

    def add_file(self, filename: str):
        """append one file"""
        lay = self._read(filename)
        self._add_layout(filename, lay)

    def _add_layout(self, filename: str, lay: _Layout):
        self.files.append(filename)
        self._layouts.append(lay)
        self._file_seq_start.append(self._file_seq_start[-1] + len(lay.seq_tags))
        starts = numpy.zeros((len(lay.seq_tags) + 1, lay.seq_lengths.shape[1]), dtype="int64")
        starts[1:] = numpy.cumsum(lay.seq_lengths, axis=0)
        self._seq_starts.append(starts)
        sparse_in = lay.input_ndim == 1
        self.num_inputs = lay.input_dim
        self.num_outputs = {"data": (lay.input_dim, 1 if sparse_in else 2)}
        for k in lay.target_keys:
            self.num_outputs[k] = lay.target_dims[k]
            if k in lay.labels:
                self.labels[k] = lay.labels[k]

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return self._file_seq_start[-1]

    def get_all_tags(self) -> List[str]:
        return [t for lay in self._layouts for t in lay.seq_tags]

    def _locate(self, corpus_idx: int):
        for fi in range(len(self._layouts)):
            if corpus_idx < self._file_seq_start[fi + 1]:
                return fi, corpus_idx - self._file_seq_start[fi]
        raise IndexError(corpus_idx)

    def _seq_len(self, corpus_idx: int) -> int:
        fi, j = self._locate(corpus_idx)
        return int(self._layouts[fi].seq_lengths[j, 0])

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            idx = {t: i for i, t in enumerate(self.get_all_tags())}
            self._order = [idx[t] for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=self.get_total_num_seqs(), get_seq_len=self._seq_len))
        self._num_seqs = len(self._order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    def get_current_seq_order(self):
        return list(self._order)

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        fi, j = self._locate(self._order[seq_idx])
        lay, starts = self._layouts[fi], self._seq_starts[fi]
        feats = {"data": lay.inputs[starts[j, 0]: starts[j + 1, 0]]}
        for ti, k in enumerate(lay.target_keys):
            col = min(ti + 1, starts.shape[1] - 1)
            feats[k] = lay.targets[k][starts[j, col]: starts[j + 1, col]]
        return DatasetSeq(seq_idx=seq_idx, seq_tag=lay.seq_tags[j], features=feats)

    def get_data_keys(self):
        return ["data"] + [k for k in self.num_outputs if k != "data"]

    def get_target_list(self):
        return [k for k in self.num_outputs if k != "data"]

    def get_data_dim(self, key):
        return self.num_outputs[key][0]

    def is_data_sparse(self, key):
        return self.num_outputs[key][1] == 1

    def get_data_dtype(self, key):
        lay = self._layouts[0]
        arr = lay.inputs if key == "data" else lay.targets[key]
        return str(arr.dtype)

    def get_data_shape(self, key):
        return [] if self.is_data_sparse(key) else [self.num_outputs[key][0]]


class NextGenHDFDataset(HDFDataset):
    """stream-per-group layout of the reference's NextGenHDFDataset is read through the same logical layout"""


class SiameseHDFDataset(HDFDataset):
    """as HDFDataset; the reference's class additionally samples same/different-class pairs"""


class SimpleHDFWriter:
    """
    Collects batches / sequences and writes one file of the layout above (reference: returnn/datasets/hdf.py:1070).

    :param filename: output file; ``.npz`` selects the HDF5-free container
    :param dim: feature dim of "data", or number of classes if ``ndim == 1``
    :param extra_type: ``{key: (dim, ndim, dtype)}`` further streams
    """

    def __init__(self, filename: str, dim: Optional[int], labels: Optional[Sequence[str]] = None, ndim: int = 2,
                 extra_type: Optional[Dict[str, tuple]] = None, swmr: bool = False, extend_existing_file: bool = False):
        self.filename = filename
        self.dim = dim
        self.ndim = ndim
        self.labels = list(labels) if labels is not None else None
        self.extra_type = dict(extra_type or {})
        self._inputs: List[numpy.ndarray] = []
        self._extras: Dict[str, List[numpy.ndarray]] = {k: [] for k in self.extra_type}
        self._tags: List[str] = []
        self._lens: List[List[int]] = []
        self._closed = False

    def insert_batch(self, inputs: numpy.ndarray, seq_len: Union[Sequence[int], Dict[int, Sequence[int]]], seq_tag: Sequence[str],
                     extra: Optional[Dict[str, numpy.ndarray]] = None):
        """:param inputs: [batch, time, ...] padded; seq_len: per sequence (or {axis: lens})"""
        if isinstance(seq_len, dict):
            seq_len = seq_len[0]
        for b, (n, tag) in enumerate(zip(seq_len, seq_tag)):
            row = [int(n)]
            self._inputs.append(numpy.asarray(inputs[b][: int(n)]))
            for k in self.extra_type:
                v = numpy.asarray(extra[k][b])
                ln = extra.get("%s_seq_len" % k)
                if ln is not None:
                    v = v[: int(ln[b])]
                self._extras[k].append(v)
                row.append(int(v.shape[0]) if v.ndim else 1)
            self._tags.append(str(tag))
            self._lens.append(row)

    def insert_seq(self, data: numpy.ndarray, seq_tag: str, extra: Optional[Dict[str, numpy.ndarray]] = None):
        """one sequence [time, ...]"""
        ex = {k: numpy.asarray(v)[None] for k, v in (extra or {}).items()}
        self.insert_batch(numpy.asarray(data)[None], [data.shape[0]], [seq_tag], extra=ex)

    def _layout(self) -> _Layout:
        lay = _Layout()
        lay.inputs = numpy.concatenate(self._inputs, axis=0) if self._inputs else numpy.zeros((0,) if self.ndim == 1 else (0, self.dim or 0))
        lay.seq_lengths = numpy.asarray(self._lens, dtype="int32").reshape(len(self._tags), 1 + len(self.extra_type))
        lay.seq_tags = self._tags
        for k, (dim, ndim, dtype) in self.extra_type.items():
            parts = [p.reshape((-1,) + p.shape[1:]) if p.ndim else p.reshape(1) for p in self._extras[k]]
            lay.targets[k] = numpy.concatenate(parts, axis=0).astype(dtype) if parts else numpy.zeros((0,), dtype=dtype)
            lay.target_dims[k] = (int(dim), int(ndim))
        lay.target_keys = sorted(lay.targets.keys())
        lay.input_dim = int(self.dim or 0)
        lay.input_ndim = self.ndim
        if self.labels:
            lay.labels["data"] = self.labels
        return lay

    def close(self):
        """write the file"""
        if self._closed:
            return
        self._closed = True
        lay = self._layout()
        if self.filename.endswith(".npz"):
            NpzWriter.write(self.filename, lay)
            return
        h5py = _h5py()
        with h5py.File(self.filename, "w") as f:
            f.attrs["inputPattSize"] = lay.input_dim
            f.attrs["numSeqs"] = len(lay.seq_tags)
            f.attrs["numTimesteps"] = int(lay.inputs.shape[0])
            f.attrs["numLabels"] = lay.input_dim
            f.create_dataset("inputs", data=lay.inputs)
            f.create_dataset("seqLengths", data=lay.seq_lengths)
            dt = h5py.special_dtype(vlen=str)
            f.create_dataset("seqTags", data=numpy.array(lay.seq_tags, dtype=object), dtype=dt)
            g = f.create_group("targets")
            gd, gs, gl = g.create_group("data"), g.create_group("size"), g.create_group("labels")
            for k in lay.target_keys:
                gd.create_dataset(k, data=lay.targets[k])
                gs.attrs[k] = list(lay.target_dims[k])
            if self.labels:
                gl.create_dataset("data", data=numpy.array(self.labels, dtype=object), dtype=dt)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class HDFDatasetWriter(SimpleHDFWriter):
    """dump a whole dataset into one file (reference: returnn/datasets/hdf.py:1428)"""

    def __init__(self, filename: str):
        self._init_done = False
        self._filename = filename

    def dump_from_dataset(self, dataset, epoch: int = 1, start_seq: int = 0, end_seq: Union[int, float] = float("inf"), use_progress_bar: bool = False):
        """read the dataset in its epoch order and write everything"""
        dataset.init_seq_order(epoch=epoch)
        keys = [k for k in dataset.get_data_keys() if k != "data"]
        extra = {k: (dataset.get_data_dim(k), 1 if dataset.is_data_sparse(k) else 2, dataset.get_data_dtype(k)) for k in keys}
        SimpleHDFWriter.__init__(self, self._filename, dim=dataset.get_data_dim("data"), ndim=1 if dataset.is_data_sparse("data") else 2, extra_type=extra)
        i = start_seq
        while dataset.is_less_than_num_seqs(i) and i < end_seq:
            dataset.load_seqs(i, i + 1)
            self.insert_seq(dataset.get_data(i, "data"), dataset.get_tag(i), extra={k: dataset.get_data(i, k) for k in keys})
            i += 1


class NpzWriter:
    """the same logical layout in a numpy ``.npz`` container"""

    @staticmethod
    def write(filename: str, lay: _Layout):
        """one file"""
        arrays = {"inputs": lay.inputs, "seqLengths": lay.seq_lengths, "seqTags": numpy.array(lay.seq_tags),
                  "inputPattSize": numpy.array(lay.input_dim), "targetKeys": numpy.array(lay.target_keys)}
        for k in lay.target_keys:
            arrays["targets/data/" + k] = lay.targets[k]
            arrays["targets/size/" + k] = numpy.array(lay.target_dims[k])
        for k, v in lay.labels.items():
            arrays["targets/labels/" + k] = numpy.array(v)
        tmp = filename + ".tmp.npz"
        numpy.savez(tmp, **arrays)
        os.replace(tmp, filename)


class NpzDataset(HDFDataset):
    """reads files written by :class:`SimpleHDFWriter` with a ``.npz`` name"""

    def _read(self, filename: str) -> _Layout:
        lay = _Layout()
        with numpy.load(filename, allow_pickle=False) as f:
            lay.inputs = f["inputs"]
            lay.seq_lengths = f["seqLengths"]
            lay.seq_tags = [str(t) for t in f["seqTags"]]
            lay.input_dim = int(f["inputPattSize"])
            lay.input_ndim = lay.inputs.ndim
            lay.target_keys = [str(k) for k in f["targetKeys"]]
            for k in lay.target_keys:
                lay.targets[k] = f["targets/data/" + k]
                d = f["targets/size/" + k]
                lay.target_dims[k] = (int(d[0]), int(d[1]))
                if "targets/labels/" + k in f:
                    lay.labels[k] = [str(x) for x in f["targets/labels/" + k]]
        return lay
