"""
:class:`HuggingFaceDataset`: a HuggingFace ``datasets.Dataset`` as a dataset of this framework. Every entry of ``data_format``
names a column that becomes a data key; string columns with a ``vocab`` are tokenised, audio columns (dicts with ``array``)
give their sample array. Sorting and shuffling by length use a length column when one is named, so that ordering an epoch does
not decode every item.  Reference: returnn/datasets/huggingface.py:24-438.

The ``datasets`` package is needed for loading by name, from disk or from Arrow files; a callable ``dataset_opts`` may also return
any object with ``__len__``, ``__getitem__(int) -> dict`` and ``__getitem__(column) -> sequence`` (what this class uses).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Union
import os
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from .util.vocabulary import Vocabulary


class _ColumnFormat:
    """dim / ndim / dtype / vocab of one data key"""

    def __init__(self, name: str, opts: Dict[str, Any]):
        opts = dict(opts)
        self.name = name
        self.vocab: Optional[Vocabulary] = None
        vocab = opts.pop("vocab", None)
        if vocab is not None:
            self.vocab = vocab if isinstance(vocab, Vocabulary) else Vocabulary.create_vocab(**vocab)
        self.sparse = bool(opts.pop("sparse", self.vocab is not None))
        shape = opts.pop("shape", None)
        self.dim = opts.pop("dim", None)
        if self.vocab is not None and self.dim is None:
            self.dim = self.vocab.num_labels
        if shape is not None:
            self.ndim = len(shape)
            if self.dim is None and not self.sparse and shape and shape[-1] is not None:
                self.dim = shape[-1]
        else:
            self.ndim = opts.pop("ndim", 1 if self.sparse else 2)
        self.dtype = opts.pop("dtype", "int32" if self.sparse else "float32")
        self.shape = list(shape) if shape is not None else ([None] * self.ndim if self.sparse else [None] * (self.ndim - 1) + [self.dim])


class HuggingFaceDataset(CachedDataset2):
    """wrapper around a HuggingFace dataset, see the module docstring"""

    def __init__(self, dataset_opts: Union[Dict[str, Any], str, os.PathLike, Sequence[Union[str, os.PathLike]], Callable[[], Any]], *,
                 use_file_cache: bool = False, map_func: Optional[Callable[[Any], Any]] = None, rename_columns: Optional[Dict[str, str]] = None,
                 cast_columns: Optional[Dict[str, Dict[str, Any]]] = None, data_format: Dict[str, Dict[str, Any]],
                 seq_tag_column: Optional[str] = "id", sorting_seq_len_column_data: Optional[str] = None,
                 sorting_seq_len_column: Optional[str] = None, **kwargs):
        super().__init__(**kwargs)
        self.dataset_opts = dataset_opts
        self.use_file_cache = use_file_cache
        self.map_func = map_func
        self.rename_columns = rename_columns
        self.cast_columns = cast_columns
        self.data_format: Dict[str, _ColumnFormat] = {k: _ColumnFormat(k, v) for k, v in data_format.items()}
        self.seq_tag_column = seq_tag_column
        self.sorting_seq_len_column_data = sorting_seq_len_column_data
        self.sorting_seq_len_column = sorting_seq_len_column
        self.labels = {k: list(f.vocab.labels) for k, f in self.data_format.items() if f.vocab is not None}
        self.num_outputs = {k: (f.dim or 1, f.ndim) for k, f in self.data_format.items()}
        self.hf_dataset: Any = None
        self._seq_order: Optional[Sequence[int]] = None
        self._seq_tags: Optional[List[str]] = None
        self._sorting_lens: Optional[Sequence[int]] = None

    def _lazy_init(self):
        if self.hf_dataset is not None:
            return
        opts = self.dataset_opts() if callable(self.dataset_opts) else self.dataset_opts
        if self.use_file_cache:
            assert isinstance(opts, (str, os.PathLike, list, tuple)), "%s: use_file_cache needs a path or a list of Arrow files" % self
            from ..utils import file_cache

            if isinstance(opts, (str, os.PathLike)):
                opts = sorted(os.path.join(os.fspath(opts), f) for f in os.listdir(os.fspath(opts)) if f.endswith(".arrow"))
            cache = file_cache.get_instance()
            opts = [cache.get_file(os.fspath(fn)) for fn in opts]
        if isinstance(opts, (dict, str, os.PathLike, list, tuple)):
            try:
                import datasets
            except ImportError as exc:
                raise ImportError("%s: loading by name or from files needs the HuggingFace `datasets` package (%s); a callable "
                                  "dataset_opts can return a dataset object directly" % (self, exc))
            if isinstance(opts, dict):
                ds = datasets.load_dataset(**opts)
            elif isinstance(opts, (str, os.PathLike)):
                ds = datasets.load_from_disk(os.fspath(opts))
            else:
                ds = datasets.concatenate_datasets([datasets.Dataset.from_file(os.fspath(fn)) for fn in opts])
        else:
            ds = opts
        assert hasattr(ds, "__len__") and hasattr(ds, "__getitem__"), "%s: expected one dataset, got %r (give the split)" % (self, type(ds))
        if self.map_func is not None:
            ds = self.map_func(ds)
        if self.rename_columns:
            ds = ds.rename_columns(self.rename_columns)
        if self.cast_columns:
            import datasets

            feats = ds.features.copy()
            for col, spec in self.cast_columns.items():
                feats[col] = datasets.features.features.generate_from_dict(spec) if isinstance(spec, dict) else spec
            ds = ds.cast(feats)
        self.hf_dataset = ds

    # -- static information
    def get_data_keys(self) -> List[str]:
        return list(self.data_format.keys())

    def get_target_list(self) -> List[str]:
        return self.get_data_keys()

    def get_data_shape(self, key: str) -> List[int]:
        f = self.data_format[key]
        return [] if f.ndim <= 1 else list(f.shape[1:])

    def get_data_dim(self, key: str) -> int:
        return self.data_format[key].dim or 1

    def is_data_sparse(self, key: str) -> bool:
        return self.data_format[key].sparse

    def get_data_dtype(self, key: str) -> str:
        return self.data_format[key].dtype

    def supports_sharding(self) -> bool:
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    # -- order
    def _get_seq_len(self, seq_idx: int) -> int:
        if self._sorting_lens is None:
            self._lazy_init()
            if self.sorting_seq_len_column:
                self._sorting_lens = [int(v) for v in self.hf_dataset[self.sorting_seq_len_column]]
            elif self.sorting_seq_len_column_data:
                self._sorting_lens = [len(v) for v in self.hf_dataset[self.sorting_seq_len_column_data]]
            else:
                raise ValueError("%s: orderings by length need sorting_seq_len_column or sorting_seq_len_column_data" % self)
        return self._sorting_lens[seq_idx]

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        self._lazy_init()
        return len(self.hf_dataset)

    def get_all_tags(self) -> List[str]:
        if self._seq_tags is None:
            self._lazy_init()
            if self.seq_tag_column:
                self._seq_tags = [str(t) for t in self.hf_dataset[self.seq_tag_column]]
            else:
                self._seq_tags = ["seq-%i" % i for i in range(len(self.hf_dataset))]
        return self._seq_tags

    def init_seq_order(self, epoch: Optional[int] = None, seq_list: Optional[Sequence[str]] = None, seq_order: Optional[Sequence[int]] = None) -> bool:
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._seq_order = list(seq_order)
        elif seq_list is not None:
            by_tag = {t: i for i, t in enumerate(self.get_all_tags())}
            self._seq_order = [by_tag[t] for t in seq_list]
        elif epoch is None:
            self._seq_order = []
        else:
            self._lazy_init()
            self._seq_order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self.hf_dataset), get_seq_len=self._get_seq_len))
        self._num_seqs = len(self._seq_order)
        return True

    @property
    def num_seqs(self) -> int:
        assert self._seq_order is not None, "%s: init_seq_order was not called" % self
        return len(self._seq_order)

    def get_current_seq_order(self) -> Sequence[int]:
        return list(self._seq_order or [])

    def get_corpus_seq_idx(self, sorted_seq_idx: int) -> int:
        return int(self._seq_order[sorted_seq_idx])

    def get_tag(self, sorted_seq_idx: int) -> str:
        return self.get_all_tags()[self.get_corpus_seq_idx(sorted_seq_idx)]

    # -- data
    def _convert(self, key: str, value) -> numpy.ndarray:
        f = self.data_format[key]
        if isinstance(value, dict) and "array" in value:  # an audio feature
            value = value["array"]
        if isinstance(value, str):
            assert f.vocab is not None, "%s: column %r holds text, give a vocab in data_format" % (self, key)
            value = f.vocab.get_seq(value)
        arr = numpy.asarray(value, dtype=f.dtype)
        if arr.ndim < f.ndim:
            arr = arr.reshape(arr.shape + (1,) * (f.ndim - arr.ndim))
        return arr

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._seq_order):
            return None
        self._lazy_init()
        corpus_idx = int(self._seq_order[seq_idx])
        item = self.hf_dataset[corpus_idx]
        feats = {k: self._convert(k, item[k]) for k in self.data_format}
        tag = str(item[self.seq_tag_column]) if self.seq_tag_column else "seq-%i" % corpus_idx
        return DatasetSeq(seq_idx=seq_idx, seq_tag=tag, features=feats)
