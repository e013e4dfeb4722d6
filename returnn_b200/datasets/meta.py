"""
Datasets built from other datasets (reference: returnn/datasets/meta.py).

- :class:`MetaDataset`: several datasets with the same sequences (matched by tag) joined into one set of data keys
  (``data_map = {key: (dataset_name, dataset_key)}``); one dataset controls the sequence order.
- :class:`CombinedDataset`: several datasets with different sequences mixed into one stream, data keys mapped through
  ``data_map = {(dataset_name, dataset_key): key}``; sampling by size or by ``sampling_sizes``.
- :class:`ConcatDataset`: datasets one after the other.
- :class:`ConcatSeqsDataset`: several sequences of a sub dataset concatenated into one (tags joined by ``;``).
- :class:`MultiEpochDataset`, :class:`VariableDataset`, :class:`AnythingDataset`, :class:`EpochWiseFilter` helper.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union
import numpy
from .basic import Dataset, DatasetSeq, init_dataset, convert_data_dims
from .cached2 import CachedDataset2
from ..utils.basic import NumbersDict
from ..log import log


class EpochWiseFilter:
    """
    ``{(ep_start, ep_end): {"max_mean_len": n}}``: in these epochs only sequences up to that length are used
    (reference: returnn/datasets/meta.py:38-140).
    """

    def __init__(self, epochs_opts: Dict[Tuple[int, Optional[int]], Dict[str, Any]], debug_msg_prefix: str = "EpochWiseFilter"):
        self.epochs_opts = epochs_opts
        self.debug_msg_prefix = debug_msg_prefix

    @classmethod
    def filter_epoch(cls, opts: Dict[str, Any], seq_order: Sequence[int], get_seq_len: Callable[[int], int], debug_msg_prefix: str) -> List[int]:
        """apply one option set"""
        opts = dict(opts)
        order = list(seq_order)
        if opts.get("max_mean_len"):
            max_mean_len = opts.pop("max_mean_len")
            lens = numpy.array(sorted(get_seq_len(i) for i in order))
            best_num = len(lens)
            csum = numpy.cumsum(lens)
            for n in range(len(lens), 0, -1):
                if csum[n - 1] / n <= max_mean_len:
                    best_num = n
                    break
            else:
                best_num = 0
            limit = lens[best_num - 1] if best_num > 0 else 0
            before = len(order)
            order = [i for i in order if get_seq_len(i) <= limit]
            print("%s, max_mean_len %s: %i -> %i seqs (max len %i)" % (debug_msg_prefix, max_mean_len, before, len(order), limit), file=log.v4)
        else:
            opts.pop("max_mean_len", None)
        if opts.get("max_len"):
            m = opts.pop("max_len")
            order = [i for i in order if get_seq_len(i) <= m]
        assert not {k: v for k, v in opts.items() if v}, "EpochWiseFilter: unknown options %r" % opts
        return order

    def filter(self, epoch: Optional[int], seq_order: Sequence[int], get_seq_len: Callable[[int], int]) -> List[int]:
        """filter for this epoch"""
        epoch = epoch or 1
        order = list(seq_order)
        for (ep_start, ep_end), opts in sorted(self.epochs_opts.items(), key=lambda kv: kv[0][0]):
            if ep_end is None or ep_end == -1:
                ep_end = 2 ** 31
            if ep_start <= epoch <= ep_end:
                order = self.filter_epoch(opts, order, get_seq_len, "%s, epoch %i" % (self.debug_msg_prefix, epoch))
        return order


class MetaDataset(CachedDataset2):
    """join the data keys of several datasets over the same sequences (reference: returnn/datasets/meta.py:143-640)"""

    def __init__(self, datasets: Dict[str, Union[Dict[str, Any], Dataset]], data_map: Dict[str, Tuple[str, str]],
                 seq_list_file: Optional[Union[str, Dict[str, str]]] = None, seq_order_control_dataset: Optional[str] = None,
                 seq_lens_file: Optional[str] = None, data_dims: Optional[Dict[str, Any]] = None, data_dtypes: Optional[Dict[str, str]] = None,
                 **kwargs):
        super().__init__(**kwargs)
        assert self.shuffle_frames_of_nseqs == 0
        self.data_map = {k: tuple(v) for k, v in data_map.items()}
        self.dataset_keys = sorted(datasets.keys())
        if "data" not in self.data_map and "data" in self.dataset_keys:
            pass
        self.seq_order_control_dataset = seq_order_control_dataset
        shared = {}
        if self.seq_order_control_dataset is None:
            shared = dict(seq_ordering=self.seq_ordering, partition_epoch=self.partition_epoch)
        self.datasets: Dict[str, Dataset] = {}
        for name, opts in datasets.items():
            if isinstance(opts, Dataset):
                self.datasets[name] = opts
            else:
                self.datasets[name] = init_dataset(opts, extra_kwargs={"name": "%s_%s" % (self.name, name)}, parent_dataset=self)
        self._seq_list_file = seq_list_file
        self.seq_list_original = self._load_seq_list(seq_list_file)
        self.num_total_seqs = len(self.seq_list_original[self.dataset_keys[0]]) if self.seq_list_original else None
        self.tag_idx: Optional[Dict[str, int]] = None
        self._seq_lens: Optional[Dict[str, NumbersDict]] = None
        if seq_lens_file:
            import ast

            raw = ast.literal_eval(open(seq_lens_file).read())
            self._seq_lens = {tag: NumbersDict(v) for tag, v in raw.items()}
        if data_dims:
            self.data_dims = convert_data_dims(data_dims)
        else:
            self.data_dims = {}
            for key, (ds_name, ds_key) in self.data_map.items():
                ds = self.datasets[ds_name]
                self.data_dims[key] = (ds.get_data_dim(ds_key), len(ds.get_data_shape(ds_key)) + 1 if not ds.is_data_sparse(ds_key) else 1)
        self.data_dtypes = {key: (data_dtypes or {}).get(key) or self.datasets[ds].get_data_dtype(k) for key, (ds, k) in self.data_map.items()}
        self.num_inputs = self.data_dims["data"][0] if "data" in self.data_dims else 0
        self.num_outputs = self.data_dims
        self.orig_seq_order_is_initialized = False
        self.seq_list_ordered: Optional[Dict[str, List[str]]] = None

    def _load_seq_list(self, seq_list_file) -> Optional[Dict[str, List[str]]]:
        if not seq_list_file:
            # all datasets must list their tags; the control dataset (or the first) defines the set
            ctrl = self.seq_order_control_dataset or self.dataset_keys[0]
            try:
                tags = self.datasets[ctrl].get_all_tags()
            except Exception:
                return None
            return {name: list(tags) for name in self.dataset_keys}
        if isinstance(seq_list_file, dict):
            lists = {name: self._read_list(fn) for name, fn in seq_list_file.items()}
            for name in self.dataset_keys:
                lists.setdefault(name, next(iter(lists.values())))
            return lists
        tags = self._read_list(seq_list_file)
        return {name: tags for name in self.dataset_keys}

    @staticmethod
    def _read_list(fn: str) -> List[str]:
        if fn.endswith(".pkl"):
            import pickle

            return list(pickle.load(open(fn, "rb")))
        opener = open
        if fn.endswith(".gz"):
            import gzip

            opener = gzip.open
        return [line.strip() for line in opener(fn, "rt").read().splitlines() if line.strip()]

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        ctrl = self.seq_order_control_dataset
        if seq_order is not None:
            order = list(seq_order)
            self.seq_list_ordered = {name: [lst[i] for i in order] for name, lst in self.seq_list_original.items()}
        elif seq_list is not None:
            self.seq_list_ordered = {name: list(seq_list) for name in self.dataset_keys}
        elif ctrl:
            ds = self.datasets[ctrl]
            ds.init_seq_order(epoch=epoch)
            try:
                order = list(ds.get_current_seq_order())
                self.seq_list_ordered = {name: [lst[i] for i in order] for name, lst in self.seq_list_original.items()}
            except Exception:
                tags = []
                i = 0
                while ds.is_less_than_num_seqs(i):
                    ds.load_seqs(i, i + 1)
                    tags.append(ds.get_tag(i))
                    i += 1
                self.seq_list_ordered = {name: tags for name in self.dataset_keys}
        else:
            assert self.seq_list_original is not None, "%s: need seq_list_file or a dataset that can list its tags" % self
            n = len(self.seq_list_original[self.dataset_keys[0]])
            get_len = None
            if self._seq_lens:
                tags0 = self.seq_list_original[self.dataset_keys[0]]
                get_len = lambda i: int(self._seq_lens[tags0[i]].max_value())  # noqa: E731
            order = self.get_seq_order_for_epoch(epoch=epoch, num_seqs=n, get_seq_len=get_len)
            self.seq_list_ordered = {name: [lst[i] for i in order] for name, lst in self.seq_list_original.items()}
        self._num_seqs = len(self.seq_list_ordered[self.dataset_keys[0]])
        for name, ds in self.datasets.items():
            if name == ctrl and seq_list is None and seq_order is None:
                continue
            ds.init_seq_order(epoch=epoch, seq_list=self.seq_list_ordered[name])
        return True

    def supports_seq_order_sorting(self) -> bool:
        if self.seq_order_control_dataset:
            return self.datasets[self.seq_order_control_dataset].supports_seq_order_sorting()
        return bool(self._seq_lens)

    def get_all_tags(self) -> List[str]:
        return list(self.seq_list_original[self.dataset_keys[0]])

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self.seq_list_original[self.dataset_keys[0]])

    def finish_epoch(self, *, free_resources: bool = False):
        super().finish_epoch(free_resources=free_resources)
        for ds in self.datasets.values():
            ds.finish_epoch(free_resources=free_resources)

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= self._num_seqs:
            return None
        tag = self.seq_list_ordered[self.dataset_keys[0]][seq_idx]
        features = {}
        for name, ds in self.datasets.items():
            ds.load_seqs(seq_idx, seq_idx + 1)
            got = ds.get_tag(seq_idx)
            want = self.seq_list_ordered[name][seq_idx]
            assert got == want, "%s: dataset %r gave tag %r, expected %r at seq %i" % (self, name, got, want, seq_idx)
        for key, (ds_name, ds_key) in self.data_map.items():
            features[key] = self.datasets[ds_name].get_data(seq_idx, ds_key)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=tag, features=features)

    def get_data_keys(self) -> List[str]:
        return sorted(self.data_map.keys())

    def get_target_list(self) -> List[str]:
        return [k for k in self.get_data_keys() if k != "data"]

    def get_data_shape(self, key: str) -> List[int]:
        ds_name, ds_key = self.data_map[key]
        return self.datasets[ds_name].get_data_shape(ds_key)

    def get_data_dtype(self, key: str) -> str:
        return self.data_dtypes[key]

    def is_data_sparse(self, key: str) -> bool:
        ds_name, ds_key = self.data_map[key]
        return self.datasets[ds_name].is_data_sparse(ds_key)

    def get_data_dim(self, key: str) -> int:
        return self.data_dims[key][0]


class ConcatDataset(CachedDataset2):
    """the sequences of several datasets one after the other (reference: returnn/datasets/meta.py:ConcatDataset)"""

    def __init__(self, datasets: Sequence[Union[Dict[str, Any], Dataset]], **kwargs):
        super().__init__(**kwargs)
        self.datasets = [d if isinstance(d, Dataset) else init_dataset(d, parent_dataset=self) for d in datasets]
        assert self.datasets
        first = self.datasets[0]
        self.num_inputs = first.num_inputs
        self.num_outputs = first.num_outputs
        self.labels = first.labels
        self._cur = 0
        self._offset = 0

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        assert seq_list is None and seq_order is None, "%s: explicit seq order not supported" % self
        super().init_seq_order(epoch=epoch)
        self._cur, self._offset = 0, 0
        for ds in self.datasets:
            ds.init_seq_order(epoch=epoch)
        return True

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        while self._cur < len(self.datasets):
            ds = self.datasets[self._cur]
            sub_idx = seq_idx - self._offset
            assert sub_idx >= 0, "%s: sequences must be requested in order" % self
            if ds.is_less_than_num_seqs(sub_idx):
                ds.load_seqs(sub_idx, sub_idx + 1)
                feats = {k: ds.get_data(sub_idx, k) for k in ds.get_data_keys()}
                return DatasetSeq(seq_idx=seq_idx, seq_tag=ds.get_tag(sub_idx), features=feats)
            self._offset += sub_idx
            self._cur += 1
        return None

    @property
    def num_seqs(self) -> int:
        return sum(ds.num_seqs for ds in self.datasets)

    def get_data_keys(self):
        return self.datasets[0].get_data_keys()

    def get_target_list(self):
        return self.datasets[0].get_target_list()

    def get_data_dim(self, key):
        return self.datasets[0].get_data_dim(key)

    def get_data_dtype(self, key):
        return self.datasets[0].get_data_dtype(key)

    def get_data_shape(self, key):
        return self.datasets[0].get_data_shape(key)

    def is_data_sparse(self, key):
        return self.datasets[0].is_data_sparse(key)


class CombinedDataset(CachedDataset2):
    """
    Mix the sequences of several datasets (e.g. supervised + unsupervised) into one epoch
    (reference: returnn/datasets/meta.py:CombinedDataset). ``data_map`` maps ``(dataset_name, dataset_key)`` to the key
    under which the data appears; keys that a dataset does not provide come out as empty arrays.
    ``sampling_sizes``: per dataset a fixed number of sequences per epoch (continuing over epochs) instead of all.
    """

    def __init__(self, datasets: Dict[str, Union[Dict[str, Any], Dataset]], data_map: Dict[Tuple[str, str], str],
                 sampling_sizes: Optional[Union[int, Dict[str, int]]] = None, data_dims: Optional[Dict[str, Any]] = None,
                 data_dtypes: Optional[Dict[str, str]] = None, **kwargs):
        super().__init__(**kwargs)
        self.dataset_keys = sorted(datasets.keys())
        self.dataset_idx2key = dict(enumerate(self.dataset_keys))
        self.datasets = {k: (v if isinstance(v, Dataset) else init_dataset(v, parent_dataset=self)) for k, v in datasets.items()}
        self.data_map = {tuple(k): v for k, v in data_map.items()}
        self.data_keys = sorted(set(self.data_map.values()))
        if isinstance(sampling_sizes, int):
            sampling_sizes = {k: sampling_sizes for k in self.dataset_keys}
        self.sampling_sizes = sampling_sizes
        self._sampling_pos = {k: 0 for k in self.dataset_keys}
        self.target2source = {}
        for (ds_name, ds_key), key in self.data_map.items():
            self.target2source.setdefault(key, {})[ds_name] = ds_key
        if data_dims:
            self.data_dims = convert_data_dims(data_dims)
        else:
            self.data_dims = {}
            for (ds_name, ds_key), key in self.data_map.items():
                ds = self.datasets[ds_name]
                self.data_dims.setdefault(key, (ds.get_data_dim(ds_key), 1 if ds.is_data_sparse(ds_key) else len(ds.get_data_shape(ds_key)) + 1))
        self.data_dtypes = dict(data_dtypes or {})
        for (ds_name, ds_key), key in self.data_map.items():
            self.data_dtypes.setdefault(key, self.datasets[ds_name].get_data_dtype(ds_key))
        self.num_outputs = self.data_dims
        self.num_inputs = self.data_dims["data"][0] if "data" in self.data_dims else 0
        self._order: List[Tuple[int, int]] = []  # (dataset index, index in that dataset's epoch order)

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        assert seq_list is None and seq_order is None, "%s: explicit seq order not supported" % self
        super().init_seq_order(epoch=epoch)
        counts = []
        for name in self.dataset_keys:
            ds = self.datasets[name]
            ds.init_seq_order(epoch=epoch)
            n = ds.num_seqs
            if self.sampling_sizes and self.sampling_sizes.get(name):
                n = min(n, self.sampling_sizes[name]) if not self.sampling_sizes.get(name) else self.sampling_sizes[name]
            counts.append(n)
        pairs = []
        for di, name in enumerate(self.dataset_keys):
            ds_n = self.datasets[name].num_seqs
            start = self._sampling_pos[name] if (self.sampling_sizes and self.sampling_sizes.get(name)) else 0
            for j in range(counts[di]):
                pairs.append((di, (start + j) % max(ds_n, 1)))
            if self.sampling_sizes and self.sampling_sizes.get(name):
                self._sampling_pos[name] = (start + counts[di]) % max(ds_n, 1)
        total = len(pairs)
        order = self.get_seq_order_for_epoch(epoch=epoch, num_seqs=total, get_seq_len=lambda i: self._pair_len(pairs[i]))
        # within one dataset the sub-sequence indices must increase (datasets are streamed): keep the interleaving, sort inside
        chosen = [pairs[i] for i in order]
        per_ds = {di: sorted(j for d, j in chosen if d == di) for di in range(len(self.dataset_keys))}
        pos = {di: 0 for di in per_ds}
        self._order = []
        for d, _ in chosen:
            self._order.append((d, per_ds[d][pos[d]]))
            pos[d] += 1
        self._num_seqs = total
        return True

    def _pair_len(self, pair) -> int:
        di, j = pair
        ds = self.datasets[self.dataset_idx2key[di]]
        try:
            return int(ds.get_seq_length(j).max_value())
        except Exception:
            return 1

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        di, j = self._order[seq_idx]
        name = self.dataset_idx2key[di]
        ds = self.datasets[name]
        ds.load_seqs(j, j + 1)
        feats = {}
        for key in self.data_keys:
            src = self.target2source[key].get(name)
            if src is not None:
                feats[key] = ds.get_data(j, src)
            else:
                dim, ndim = self.data_dims[key]
                shape = (0,) if ndim == 1 else (0, dim)
                feats[key] = numpy.zeros(shape, dtype=self.data_dtypes[key])
        return DatasetSeq(seq_idx=seq_idx, seq_tag=ds.get_tag(j), features=feats)

    def get_data_keys(self):
        return list(self.data_keys)

    def get_target_list(self):
        return [k for k in self.data_keys if k != "data"]

    def get_data_dim(self, key):
        return self.data_dims[key][0]

    def get_data_dtype(self, key):
        return self.data_dtypes[key]

    def is_data_sparse(self, key):
        return self.data_dims[key][1] == 1 and self.data_dtypes[key].startswith("int")

    def get_data_shape(self, key):
        dim, ndim = self.data_dims[key]
        return [] if ndim == 1 else [dim]


class ConcatSeqsDataset(CachedDataset2):
    """
    Sequences of the sub dataset joined along time into longer ones; ``seq_list_file`` has one new sequence per line,
    the original tags separated by ``;`` (reference: returnn/datasets/meta.py:ConcatSeqsDataset).
    ``seq_len_file`` maps original tags to lengths (for sorting); ``repeat_in_between_last_frame_up_to_multiple_of``
    pads every part except the last to a multiple by repeating its last frame.
    """

    def __init__(self, dataset: Union[Dict[str, Any], Dataset], seq_list_file: str, seq_len_file: Optional[str] = None, seq_tag_delim: str = ";",
                 remove_in_between_postfix: Optional[Dict[str, int]] = None,
                 repeat_in_between_last_frame_up_to_multiple_of: Optional[Dict[str, int]] = None, use_cache_manager: bool = False,
                 epoch_wise_filter: Optional[Dict] = None, **kwargs):
        super().__init__(**kwargs)
        self.seq_tag_delim = seq_tag_delim
        self.remove_in_between_postfix = remove_in_between_postfix or {}
        self.repeat_multiple = repeat_in_between_last_frame_up_to_multiple_of or {}
        self.epoch_wise_filter = EpochWiseFilter(epoch_wise_filter) if epoch_wise_filter else None
        self.dataset = dataset if isinstance(dataset, Dataset) else init_dataset(dataset, parent_dataset=self)
        self.num_inputs = self.dataset.num_inputs
        self.num_outputs = self.dataset.num_outputs
        self.labels = self.dataset.labels
        self.full_seq_list = MetaDataset._read_list(seq_list_file)
        self.seq_lens = None
        if seq_len_file:
            import ast

            self.seq_lens = ast.literal_eval(open(seq_len_file).read())
        self.cur_seq_list: List[str] = []
        self.cur_sub_seq_idxs: List[List[int]] = []

    def _full_len(self, i: int) -> int:
        return sum(self.seq_lens[t] for t in self.full_seq_list[i].split(self.seq_tag_delim))

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            order = list(seq_order)
        elif seq_list is not None:
            idx = {t: i for i, t in enumerate(self.full_seq_list)}
            order = [idx[t] for t in seq_list]
        else:
            order = self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self.full_seq_list), get_seq_len=self._full_len if self.seq_lens else None)
            if self.epoch_wise_filter:
                order = self.epoch_wise_filter.filter(epoch=epoch, seq_order=order, get_seq_len=self._full_len)
        self.cur_seq_list = [self.full_seq_list[i] for i in order]
        sub_list, self.cur_sub_seq_idxs = [], []
        for tag in self.cur_seq_list:
            parts = tag.split(self.seq_tag_delim)
            self.cur_sub_seq_idxs.append(list(range(len(sub_list), len(sub_list) + len(parts))))
            sub_list.extend(parts)
        self.dataset.init_seq_order(epoch=epoch, seq_list=sub_list)
        self._num_seqs = len(self.cur_seq_list)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return self.seq_lens is not None

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self.cur_seq_list):
            return None
        idxs = self.cur_sub_seq_idxs[seq_idx]
        self.dataset.load_seqs(idxs[0], idxs[-1] + 1)
        feats = {}
        for key in self.dataset.get_data_keys():
            parts = []
            for n, j in enumerate(idxs):
                d = self.dataset.get_data(j, key)
                if n < len(idxs) - 1:
                    cut = self.remove_in_between_postfix.get(key)
                    if cut:
                        d = d[:-cut]
                    mult = self.repeat_multiple.get(key)
                    if mult and d.shape[0] % mult:
                        d = numpy.concatenate([d] + [d[-1:]] * (mult - d.shape[0] % mult), axis=0)
                parts.append(d)
            feats[key] = numpy.concatenate(parts, axis=0)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=self.cur_seq_list[seq_idx], features=feats)

    def get_data_keys(self):
        return self.dataset.get_data_keys()

    def get_target_list(self):
        return self.dataset.get_target_list()

    def get_data_dim(self, key):
        return self.dataset.get_data_dim(key)

    def get_data_dtype(self, key):
        return self.dataset.get_data_dtype(key)

    def get_data_shape(self, key):
        return self.dataset.get_data_shape(key)

    def is_data_sparse(self, key):
        return self.dataset.is_data_sparse(key)


class _WrapOne(CachedDataset2):
    """shared plumbing of the single-dataset wrappers below"""

    dataset: Dataset

    def _adopt(self, ds: Dataset):
        self.dataset = ds
        self.num_inputs, self.num_outputs, self.labels = ds.num_inputs, ds.num_outputs, ds.labels

    def get_data_keys(self):
        return self.dataset.get_data_keys()

    def get_target_list(self):
        return self.dataset.get_target_list()

    def get_data_dim(self, key):
        return self.dataset.get_data_dim(key)

    def get_data_dtype(self, key):
        return self.dataset.get_data_dtype(key)

    def get_data_shape(self, key):
        return self.dataset.get_data_shape(key)

    def is_data_sparse(self, key):
        return self.dataset.is_data_sparse(key)

    @property
    def num_seqs(self) -> int:
        return self.dataset.num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        ds = self.dataset
        if not ds.is_less_than_num_seqs(seq_idx):
            return None
        ds.load_seqs(seq_idx, seq_idx + 1)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=ds.get_tag(seq_idx), features={k: ds.get_data(seq_idx, k) for k in ds.get_data_keys()})


class MultiEpochDataset(_WrapOne):
    """
    One epoch here covers ``multi_epoch`` epochs of the sub dataset: the reverse of ``partition_epoch``, for sub datasets
    whose own epoch is a fraction of the data (reference: returnn/datasets/meta.py:MultiEpochDataset).
    """

    def __init__(self, dataset: Union[Dict[str, Any], Dataset], multi_epoch: int, **kwargs):
        super().__init__(**kwargs)
        assert multi_epoch >= 1
        self.multi_epoch = multi_epoch
        self._adopt(dataset if isinstance(dataset, Dataset) else init_dataset(dataset, parent_dataset=self))
        self._sub_ep = 0
        self._offset = 0

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        assert seq_list is None and seq_order is None
        super().init_seq_order(epoch=epoch)
        self._sub_ep, self._offset = 0, 0
        self.dataset.init_seq_order(epoch=((epoch or 1) - 1) * self.multi_epoch + 1)
        return True

    @property
    def num_seqs(self) -> int:
        raise NotImplementedError("%s: the number of sequences is only known at the end" % self)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        while True:
            sub = seq_idx - self._offset
            if self.dataset.is_less_than_num_seqs(sub):
                self.dataset.load_seqs(sub, sub + 1)
                ds = self.dataset
                return DatasetSeq(seq_idx=seq_idx, seq_tag=ds.get_tag(sub), features={k: ds.get_data(sub, k) for k in ds.get_data_keys()})
            self._sub_ep += 1
            if self._sub_ep >= self.multi_epoch:
                return None
            self._offset = seq_idx
            self.dataset.init_seq_order(epoch=((self.epoch or 1) - 1) * self.multi_epoch + 1 + self._sub_ep)


class VariableDataset(_WrapOne):
    """the dataset is built anew every epoch by ``get_dataset(epoch=..., **_)`` (reference: returnn/datasets/meta.py:VariableDataset)"""

    def __init__(self, get_dataset: Callable[..., Union[Dict[str, Any], Dataset]], dataset_lru_cache_size: int = 1, always_same_tags: bool = False,
                 **kwargs):
        super().__init__(**kwargs)
        self._get_dataset = get_dataset
        self.always_same_tags = always_same_tags
        self._cache: Dict[str, Dataset] = {}
        self._cache_size = dataset_lru_cache_size
        self._load(1)

    def _load(self, epoch: int):
        from ..utils.basic import get_fwd_compat_kwargs

        d = self._get_dataset(self=self, epoch=epoch, **get_fwd_compat_kwargs())
        if isinstance(d, Dataset):
            self._adopt(d)
            return
        key = repr(d)
        ds = self._cache.pop(key, None)
        if ds is None:
            ds = init_dataset(d, parent_dataset=self)
        self._cache[key] = ds
        while len(self._cache) > max(self._cache_size, 1):
            self._cache.pop(next(iter(self._cache)))
        self._adopt(ds)

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        self._load(epoch or 1)
        self.dataset.init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        return True

    def get_all_tags(self):
        return self.dataset.get_all_tags()


class ClusteringDataset(_WrapOne):
    """
    One sub-dataset plus a cluster index per sequence (data key ``cluster_idx``, one int32), read from a cluster-map file in the
    Sprint XML format: lines ``<map-item key="<seq tag>" value="<cluster>"/>`` inside ``<coprus-key-map>`` (spelled like that in those
    files). ``single_cluster``: the legacy batch generator keeps every batch within one cluster.
    Reference: returnn/datasets/meta.py:642-760.
    """

    def __init__(self, dataset: Dict[str, Any], cluster_map_file: str, n_clusters: int, single_cluster: bool = False, **kwargs):
        super().__init__(**kwargs)
        self._adopt(init_dataset(dataset, parent_dataset=self))
        self.n_clusters = n_clusters
        self.single_cluster = single_cluster
        self.cluster_idx_dtype = "int32"
        self.cluster_map = self._load_cluster_map(cluster_map_file)
        self.num_outputs = dict(self.dataset.num_outputs)
        self.num_outputs["cluster_idx"] = (n_clusters, 1)

    def _load_cluster_map(self, filename: str) -> Dict[str, int]:
        import re

        with open(filename) as f:
            lines = f.read().splitlines()
        assert any("<coprus-key-map>" in ln or "<corpus-key-map>" in ln for ln in lines[:3]), "%s: expected the Sprint XML cluster-map format" % filename
        item = re.compile(r'\s*<map-item key="(.*)" value="(.*)"/>')
        out: Dict[str, int] = {}
        for ln in lines:
            m = item.match(ln)
            if m:
                idx = int(m.group(2))
                assert 0 <= idx < self.n_clusters, "%s: cluster %i outside 0..%i" % (filename, idx, self.n_clusters - 1)
                out[m.group(1)] = idx
        return out

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        self.dataset.init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        return super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)

    def get_data_keys(self):
        return list(self.dataset.get_data_keys()) + ["cluster_idx"]

    def get_data_dtype(self, key):
        return self.cluster_idx_dtype if key == "cluster_idx" else self.dataset.get_data_dtype(key)

    def get_data_dim(self, key):
        return self.n_clusters if key == "cluster_idx" else self.dataset.get_data_dim(key)

    def get_data_shape(self, key):
        return [] if key == "cluster_idx" else self.dataset.get_data_shape(key)

    def is_data_sparse(self, key):
        return True if key == "cluster_idx" else self.dataset.is_data_sparse(key)

    def is_less_than_num_seqs(self, n):
        return self.dataset.is_less_than_num_seqs(n)

    def get_tag(self, seq_idx):
        return self.dataset.get_tag(seq_idx)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        seq = super()._collect_single_seq(seq_idx)
        if seq is None:
            return None
        seq.features["cluster_idx"] = numpy.array([self.cluster_map[seq.seq_tag]], dtype=self.cluster_idx_dtype)
        return seq

    def _generate_batches(self, recurrent_net, batch_size, max_seqs=-1, seq_drop=0.0, max_seq_length=None, used_data_keys=None, **kwargs):
        if not self.single_cluster:
            yield from super()._generate_batches(recurrent_net=recurrent_net, batch_size=batch_size, max_seqs=max_seqs, seq_drop=seq_drop,
                                                 max_seq_length=max_seq_length if max_seq_length is not None else 2 ** 31,
                                                 used_data_keys=used_data_keys, **kwargs)
            return
        from ..engine.batch import Batch

        budget = NumbersDict(batch_size or 2 ** 31)
        limit = NumbersDict(max_seq_length if max_seq_length is not None else 2 ** 31)
        max_seqs_ = float("inf") if max_seqs == -1 else max_seqs
        batch, batch_cluster = Batch(), None
        for seq_idx, t_start, t_end in self.iterate_seqs(recurrent_net=recurrent_net, used_data_keys=used_data_keys):
            length = t_end - t_start
            if length.any_compare(limit, (lambda a, b: a > b)):
                continue
            if self.rnd_seq_drop.random_sample() < seq_drop:
                continue
            cluster = self.cluster_map[self.get_tag(seq_idx)]
            dt, ds = batch.try_sequence_as_slice(length)
            full = batch.num_slices >= 1 and ((dt * ds).any_compare(budget, (lambda a, b: a > b)) or ds > max_seqs_)
            if batch.num_slices >= 1 and (full or cluster != batch_cluster):
                yield batch
                batch = Batch()
            batch_cluster = cluster
            batch.add_sequence_as_slice(seq_idx=seq_idx, seq_start_frame=t_start, length=length)
        if batch.num_slices:
            yield batch


class ChunkShuffleDataset(CachedDataset2):
    """
    Chunks (the batches of the sub-dataset's legacy batch generator, ``batch_gen_max_seqs`` sequences or chunks each) turned into
    sequences of their own and shuffled within a sliding cache of ``chunk_shuffle_cache`` chunks: a cheap way to decorrelate
    neighbouring chunks of long recordings without loading everything. Tags: ``<original tag>.<running index>``.
    Reference: returnn/datasets/meta.py:1873-2010.
    """

    def __init__(self, dataset: Dict[str, Any], chunk_shuffle_cache: int = 1000, batch_gen_batch_size: int = 5000, batch_gen_max_seqs: int = 1,
                 batch_gen_recurrent_net: bool = True, **kwargs):
        super().__init__(**kwargs)
        import random

        self.dataset = init_dataset(dataset, parent_dataset=self)
        self.chunk_shuffle_cache = chunk_shuffle_cache
        self.batch_gen_batch_size = batch_gen_batch_size
        self.batch_gen_max_seqs = batch_gen_max_seqs
        self.batch_gen_recurrent_net = batch_gen_recurrent_net
        self.num_inputs, self.num_outputs, self.labels = self.dataset.num_inputs, self.dataset.num_outputs, self.dataset.labels
        self.rng = random.Random(0)
        self._batches = None
        self._pool: List[DatasetSeq] = []  # chunks read from the sub-dataset and not handed out yet
        self._made = 0  # chunks read so far
        self._exhausted = False
        self._last_loaded_end = 0

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        if seq_list is not None or seq_order is not None:
            raise NotImplementedError("%s: a predefined order is not supported" % self)
        if self.seq_ordering != "default":
            raise NotImplementedError("%s: seq_ordering %r (order the sub-dataset instead)" % (self, self.seq_ordering))
        super().init_seq_order(epoch=epoch)
        self.rng.seed(epoch or 1)
        self.dataset.init_seq_order(epoch=epoch)
        self._batches = iter(self.dataset._generate_batches(recurrent_net=self.batch_gen_recurrent_net, batch_size=self.batch_gen_batch_size,
                                                            max_seqs=self.batch_gen_max_seqs))
        self._pool, self._made, self._exhausted, self._last_loaded_end = [], 0, False, 0
        self._num_seqs = None
        return True

    def _read_chunk_batch(self) -> bool:
        batch = next(self._batches, None)
        if batch is None:
            self._exhausted = True
            return False
        if batch.end_seq > self._last_loaded_end:
            self.dataset.load_seqs(batch.start_seq, batch.end_seq)
            self._last_loaded_end = batch.end_seq
        keys = self.get_data_keys()
        for part in batch.seqs:
            feats = {}
            for k in keys:
                data = self.dataset.get_data(part.seq_idx, k)
                if data is not None:
                    feats[k] = data[part.seq_start_frame[k]: part.seq_end_frame[k]]
            self._pool.append(DatasetSeq(seq_idx=-1, seq_tag="%s.%i" % (self.dataset.get_tag(part.seq_idx), self._made), features=feats))
            self._made += 1
        return True

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        # keep the cache full, then hand out a random member of it
        while not self._exhausted and len(self._pool) < self.chunk_shuffle_cache:
            self._read_chunk_batch()
        if not self._pool:
            return None
        pick = self.rng.randrange(len(self._pool))
        seq = self._pool.pop(pick)
        seq.seq_idx = seq_idx
        return seq

    def get_data_keys(self):
        return self.dataset.get_data_keys()

    def get_target_list(self):
        return self.dataset.get_target_list()

    def get_data_dim(self, key):
        return self.dataset.get_data_dim(key)

    def get_data_dtype(self, key):
        return self.dataset.get_data_dtype(key)

    def is_data_sparse(self, key):
        return self.dataset.is_data_sparse(key)


class AnythingDataset(Dataset):
    """
    Empty dataset that only declares data keys and dims: for tasks that need ``extern_data`` but never read data
    (reference: returnn/datasets/meta.py:AnythingDataset).
    """

    def __init__(self, data_keys: Dict[str, Dict[str, Any]], **kwargs):
        super().__init__(**kwargs)
        self._data_keys = data_keys
        self.num_outputs = {k: (v.get("dim") or (v.get("shape") or [1])[-1] or 1, len(v.get("shape", ())) + (0 if v.get("sparse") else 0) or 1)
                            for k, v in data_keys.items()}
        self.num_inputs = self.num_outputs.get("data", (0, 0))[0]

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        return True

    @property
    def num_seqs(self) -> int:
        return 0

    def is_less_than_num_seqs(self, n: int) -> bool:
        return False

    def get_data_keys(self):
        return list(self._data_keys.keys())

    def get_target_list(self):
        return [k for k in self._data_keys if k != "data"]

    def get_data_dtype(self, key):
        return self._data_keys[key].get("dtype", "float32")

    def is_data_sparse(self, key):
        return bool(self._data_keys[key].get("sparse", False))

    def get_data_shape(self, key):
        return list(self._data_keys[key].get("shape", ()))[1:]

    def _load_seqs(self, start, end):
        pass
