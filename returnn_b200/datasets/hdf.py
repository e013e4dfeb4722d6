"""
HDF5 datasets and writers (reference: returnn/datasets/hdf.py).

File layout of :class:`HDFDataset` (written by :class:`SimpleHDFWriter` / :class:`HDFDatasetWriter`):
``inputs`` ``[total_frames, dim]`` (or ``[total_frames]`` when sparse), ``seqLengths`` ``[num_seqs, 1 + num_targets]``,
``seqTags`` ``[num_seqs]``, ``targets/data/<key>``, ``targets/size/<key>`` (attrs: dim, ndim), ``targets/labels/<key>``,
file attrs ``inputPattSize``, ``numSeqs``, ``numTimesteps``, ``numLabels``.

``h5py`` is an optional dependency. Without it the same code runs on the stand-in of :mod:`returnn_b200.utils.h5_shim` (same
object model; the container is then a numpy archive, not HDF5). ``NpzDataset`` / ``NpzWriter`` below keep the logical layout of
:class:`HDFDataset` in a plain ``.npz`` file.

:class:`NextGenHDFDataset` / :class:`SiameseHDFDataset` read the stream layout: ``seq_names`` plus one group per stream under
``streams`` (attr ``parser`` = feature_sequence / sparse / segment_alignment, group ``data`` with one dataset per sequence, and
``feature_names`` for the sparse kinds); :class:`NextGenHDFWriter` writes it.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Union
import os
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from ..utils.basic import NumbersDict


def _h5py():
    """h5py, or its stand-in where the package is missing"""
    from ..utils.h5_shim import get_h5py

    return get_h5py()


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


def _decode(x) -> str:
    return x.decode("utf8") if isinstance(x, bytes) else str(x)


class StreamParser:
    """
    One stream of one stream-layout file: ``get_data(seq_name)``, ``get_seq_length(seq_name)``, and after construction
    ``num_features``, ``feature_type`` (1 sparse, 2 dense) and ``dtype``. Reference: returnn/datasets/hdf.py:475-628.
    """

    feature_type = 0

    def __init__(self, seq_names: Sequence[str], stream):
        self.seq_names = list(seq_names)
        self.stream = stream
        self.num_features: Optional[int] = None
        self.dtype: Optional[str] = None
        for name in self.seq_names:
            self._check(self.stream["data"][name])

    def _check(self, seq_data):
        if self.dtype is None:
            self.dtype = str(seq_data.dtype)
        assert str(seq_data.dtype) == self.dtype, "stream with mixed dtypes: %s vs %s" % (seq_data.dtype, self.dtype)

    def get_data(self, seq_name: str) -> numpy.ndarray:
        """the sequence's array"""
        return self.stream["data"][seq_name][...]

    def get_seq_length(self, seq_name: str) -> int:
        """its length"""
        return int(self.stream["data"][seq_name].shape[0])

    def get_dtype(self) -> str:
        """numpy dtype name"""
        assert isinstance(self.dtype, str)
        return self.dtype


class FeatureSequenceStreamParser(StreamParser):
    """dense ``[time, features]`` per sequence"""

    feature_type = 2

    def _check(self, seq_data):
        super()._check(seq_data)
        assert len(seq_data.shape) == 2
        if self.num_features is None:
            self.num_features = int(seq_data.shape[1])
        assert seq_data.shape[1] == self.num_features


class SparseStreamParser(StreamParser):
    """class indices ``[time]`` per sequence; the number of classes is the length of ``feature_names``"""

    feature_type = 1

    def __init__(self, seq_names, stream):
        super().__init__(seq_names, stream)
        self.num_features = int(stream["feature_names"].shape[0])

    def _check(self, seq_data):
        super()._check(seq_data)
        assert len(seq_data.shape) == 1


class SegmentAlignmentStreamParser(StreamParser):
    """
    Segments ``[num_segments, 2]`` = (class, length) per sequence, expanded to a frame-wise alignment that is returned flattened as
    ``[2 * frames]``: (class, 1 at the last frame of a segment else 0) per frame.
    """

    feature_type = 1

    def __init__(self, seq_names, stream):
        super().__init__(seq_names, stream)
        self.num_features = int(stream["feature_names"].shape[0])

    def _check(self, seq_data):
        super()._check(seq_data)
        assert len(seq_data.shape) == 2 and seq_data.shape[1] == 2

    def get_seq_length(self, seq_name: str) -> int:
        return 2 * int(numpy.sum(self.stream["data"][seq_name][:, 1]))

    def get_data(self, seq_name: str) -> numpy.ndarray:
        segments = self.stream["data"][seq_name][...]
        frames = int(segments[:, 1].sum())
        alignment = numpy.zeros((frames, 2), dtype=self.dtype)
        ends = numpy.cumsum(segments[:, 1])
        alignment[:, 0] = numpy.repeat(segments[:, 0], segments[:, 1])
        alignment[ends[segments[:, 1] > 0] - 1, 1] = 1
        return alignment.reshape(-1)


class _StreamHDFBase(CachedDataset2):
    """what the two stream-layout datasets share: the files, the sequence index over all files, one parser per stream and file"""

    parsers = {"feature_sequence": FeatureSequenceStreamParser, "sparse": SparseStreamParser, "segment_alignment": SegmentAlignmentStreamParser}

    def __init__(self, input_stream_name: str, files: Optional[Sequence[str]] = None, **kwargs):
        super().__init__(**kwargs)
        self.input_stream_name = input_stream_name
        self.files: List[str] = []
        self.h5_files: List[Any] = []
        self.all_seq_names: List[str] = []
        self.seq_name_to_idx: Dict[str, int] = {}
        self.file_indices: List[int] = []
        self.seq_order: List[int] = []
        self.all_parsers: Dict[str, List[StreamParser]] = {}
        for fn in files or []:
            self.add_file(fn)

    @staticmethod
    def _normalize_seq_name(name: str) -> str:
        """a dataset name cannot contain '/' (it would make sub-groups): stored with a backslash instead"""
        return name.replace("/", "\\")

    def _required_streams(self) -> List[str]:
        return [self.input_stream_name]

    def add_file(self, path: str):
        """register one more file"""
        f = _h5py().File(path, "r")
        assert "seq_names" in f and "streams" in f, "%s does not contain all required datasets/groups" % path
        self.files.append(path)
        self.h5_files.append(f)
        seqs = [_decode(x) for x in f["seq_names"][...]]
        norm = [self._normalize_seq_name(x) for x in seqs]
        first = len(self.all_seq_names)
        self.seq_name_to_idx.update({name: first + i for i, name in enumerate(seqs)})
        self.all_seq_names.extend(seqs)
        self.file_indices.extend([len(self.files) - 1] * len(seqs))
        for need in self._required_streams():
            assert need in f["streams"], "%s does not contain the stream %s" % (path, need)
        parsers = {}
        for name in f["streams"].keys():
            stream = f["streams"][name]
            kind = _decode(stream.attrs["parser"])
            parsers[name] = self.parsers[kind](norm, stream)
        for name, parser in parsers.items():
            self.all_parsers.setdefault(name, []).append(parser)
        if len(self.files) == 1:
            self.num_outputs = {name: [parser.num_features, parser.feature_type] for name, parser in parsers.items()}
            self.num_inputs = self.num_outputs[self.input_stream_name][0]
        else:
            for name, parser in parsers.items():
                assert self.num_outputs[name][0] == parser.num_features, "number of features of stream %s: %s (first file) vs %s (%s)" % (
                    name, self.num_outputs[name][0], parser.num_features, path)

    def initialize(self):
        self._num_seqs = len(self.all_seq_names)
        self._estimated_num_seqs = self._num_seqs
        super().initialize()

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self.all_seq_names)

    def get_all_tags(self) -> List[str]:
        return list(self.all_seq_names)

    def _get_seq_length(self, orig_seq_idx: int) -> int:
        parser = self.all_parsers[self.input_stream_name][self.file_indices[orig_seq_idx]]
        return parser.get_seq_length(self._normalize_seq_name(self.all_seq_names[orig_seq_idx]))

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self.seq_order = list(seq_order)
        elif seq_list is not None:
            self.seq_order = [self.seq_name_to_idx[x] for x in seq_list]
        else:
            self.seq_order = list(self.get_seq_order_for_epoch(epoch or 1, len(self.all_seq_names), self._get_seq_length))
        self._num_seqs = len(self.seq_order)
        return True

    @property
    def num_seqs(self) -> int:
        return len(self.seq_order)

    def supports_seq_order_sorting(self) -> bool:
        return True

    def supports_sharding(self) -> bool:
        return True

    def get_current_seq_order(self):
        return list(self.seq_order)

    def _stream_data(self, orig_seq_idx: int) -> Dict[str, numpy.ndarray]:
        fi = self.file_indices[orig_seq_idx]
        name = self._normalize_seq_name(self.all_seq_names[orig_seq_idx])
        return {stream: parsers[fi].get_data(name) for stream, parsers in self.all_parsers.items()}

    def get_data_dtype(self, key: str) -> str:
        if key == "data":
            key = self.input_stream_name
        return self.all_parsers[key][0].get_dtype()


class NextGenHDFDataset(_StreamHDFBase):
    """
    Stream-layout HDF files: every stream of a file becomes a data key; ``"data"`` is the stream named by ``input_stream_name``.
    Reference: returnn/datasets/hdf.py:631-788.
    """

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self.seq_order):
            return None
        orig = self.seq_order[seq_idx]
        targets = self._stream_data(orig)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=self.all_seq_names[orig], features=targets[self.input_stream_name], targets=targets)


class SiameseHDFDataset(_StreamHDFBase):
    """
    Triplet sampling for weakly supervised training on stream-layout files in which every sequence has ONE label (first entry of
    its ``seq_label_stream``). Before each epoch every sequence gets a partner with the same label (itself if it is alone in its
    class) and one with a different label, drawn uniformly over the classes or by ``class_distribution`` (path to an ``.npz`` whose
    ``arr_0[i]`` holds the probabilities of the other classes for anchor class i). Data keys: ``<stream>_0`` (anchor), ``<stream>_1``
    (same label), ``<stream>_2`` (different label) for every stream, and ``<label stream>_all`` = the three labels concatenated;
    ``"data"`` is the anchor's input stream. Reference: returnn/datasets/hdf.py:791-1067.
    """

    def __init__(self, input_stream_name: str, seq_label_stream: str = "words", class_distribution: Optional[str] = None,
                 files: Optional[Sequence[str]] = None, **kwargs):
        self.targets_stream = seq_label_stream
        self.class_probs = numpy.load(class_distribution)["arr_0"] if class_distribution is not None else None
        self.seq_to_target: Dict[str, int] = {}
        self.target_to_seqs: Dict[int, List[str]] = {}
        self.curr_epoch_triplets: List[tuple] = []
        self._triplet_rng = numpy.random.RandomState()
        super().__init__(input_stream_name, files=files, **kwargs)

    def _required_streams(self) -> List[str]:
        return [self.input_stream_name] + ([self.targets_stream] if self.targets_stream is not None else [])

    def initialize(self):
        self.target_to_seqs, self.seq_to_target = {}, {}
        for fi, f in enumerate(self.h5_files):
            labels = f["streams"][self.targets_stream]["data"]
            for orig, name in enumerate(self.all_seq_names):
                if self.file_indices[orig] != fi:
                    continue
                target = int(labels[self._normalize_seq_name(name)][0])
                self.target_to_seqs.setdefault(target, []).append(name)
                self.seq_to_target[name] = target
        super().initialize()

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if not self.seq_to_target:
            self.initialize()
        # fresh partners every epoch; with a fixed_random_seed the draws repeat per epoch number
        seed = (self._get_random_seed_for_epoch(epoch or 1) + (epoch or 1)) % (2 ** 31) if self.fixed_random_seed is not None else None
        self._triplet_rng = numpy.random.RandomState(seed)
        self._init_triplets()
        return True

    def _sample_diff_class(self, anchor_target: int) -> int:
        classes = list(self.target_to_seqs.keys())
        if self.class_probs is not None:
            probs = numpy.array(self.class_probs[anchor_target][classes], dtype="float64")
            probs /= probs.sum()
            return int(self._triplet_rng.choice(classes, p=probs))
        return int(classes[self._triplet_rng.randint(0, len(classes))])

    def _init_triplets(self):
        assert len(self.target_to_seqs) > 1, "SiameseHDFDataset needs at least two classes"
        self.curr_epoch_triplets = []
        rng = self._triplet_rng
        for orig in self.seq_order:
            name = self.all_seq_names[orig]
            target = self.seq_to_target[name]
            same = self.target_to_seqs[target]
            pair = orig
            if len(same) > 1:
                while True:
                    cand = same[rng.randint(0, len(same))]
                    if cand != name:
                        break
                pair = self.seq_name_to_idx[cand]
            other = self._sample_diff_class(target)
            while other == target:
                other = self._sample_diff_class(target)
            third_names = self.target_to_seqs[other]
            third = self.seq_name_to_idx[third_names[rng.randint(0, len(third_names))]]
            self.curr_epoch_triplets.append((orig, pair, third))

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self.seq_order):
            return None
        targets: Dict[str, numpy.ndarray] = {}
        for pos, orig in enumerate(self.curr_epoch_triplets[seq_idx]):
            for stream, arr in self._stream_data(orig).items():
                targets["%s_%d" % (stream, pos)] = arr
        ts = self.targets_stream
        targets["%s_all" % ts] = numpy.concatenate([targets["%s_%d" % (ts, i)] for i in range(3)], axis=0)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=self.all_seq_names[self.seq_order[seq_idx]],
                          features=targets["%s_0" % self.input_stream_name], targets=targets)

    def get_data_keys(self):
        keys = ["data"]
        for stream in self.all_parsers:
            keys += ["%s_%d" % (stream, i) for i in range(3)]
        return keys + ["%s_all" % self.targets_stream]

    def is_data_sparse(self, key: str) -> bool:
        if key == "data":
            key = self.input_stream_name
        return "features" not in key

    def get_data_dim(self, key: str) -> int:
        if key == "data":
            return self.num_outputs[self.input_stream_name][0]
        base = "_".join(key.split("_")[:-1]) if "_" in key else key
        return self.num_outputs[base][0] if base in self.num_outputs else 1

    def get_data_dtype(self, key: str) -> str:
        if key == "data":
            key = self.input_stream_name
        base = "_".join(key.split("_")[:-1]) if key not in self.all_parsers and "_" in key else key
        return self.all_parsers[base][0].get_dtype()


class NextGenHDFWriter:
    """
    Writes the stream layout: ``add_stream(name, kind, feature_names=...)`` once per stream, then ``add_seq(seq_name, {stream:
    array})`` per sequence, then ``close()``.
    """

    def __init__(self, filename: str):
        self._h5 = _h5py()
        self._file = self._h5.File(filename, "w")
        self._streams = self._file.create_group("streams")
        self._seq_names: List[str] = []

    def add_stream(self, name: str, kind: str, feature_names: Optional[Sequence[str]] = None):
        """``kind``: feature_sequence, sparse or segment_alignment (the last two need ``feature_names``)"""
        assert kind in _StreamHDFBase.parsers
        grp = self._streams.create_group(name)
        grp.attrs["parser"] = kind
        grp.create_group("data")
        if kind != "feature_sequence":
            assert feature_names is not None, "stream %r of kind %s needs feature_names" % (name, kind)
            grp.create_dataset("feature_names", data=numpy.array(list(feature_names), dtype=object), dtype=self._h5.special_dtype(vlen=str))

    def add_seq(self, seq_name: str, data: Dict[str, numpy.ndarray]):
        """one sequence for every stream"""
        self._seq_names.append(seq_name)
        norm = _StreamHDFBase._normalize_seq_name(seq_name)
        for stream, arr in data.items():
            self._streams[stream]["data"].create_dataset(norm, data=numpy.asarray(arr))

    def close(self):
        """write ``seq_names`` and close the file"""
        self._file.create_dataset("seq_names", data=numpy.array(self._seq_names, dtype=object), dtype=self._h5.special_dtype(vlen=str))
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


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
