"""
Dataset base class and factory.

A dataset is an ordered collection of sequences; every sequence has one numpy array per data key
(``"data"``, ``"classes"``, ...). Per (sub)epoch, ``init_seq_order`` fixes the order; then the consumer iterates
``load_seqs(i, i+1)`` / ``get_data(i, key)`` with increasing ``i`` until ``is_less_than_num_seqs(i)`` is False.

Sequence orderings (``seq_ordering``): ``default``, ``default_every_n:N``, ``reverse``, ``sorted``, ``sorted_reverse``,
``random[:nth]``, ``random_sample[:nth]``, ``sort_bin_shuffle[_x2][:bins|:.binsize[:nth]]``, ``laplace[:bins|:.binsize[:nth]]``;
or a callable ``(epoch, **kwargs) -> str``. ``partition_epoch`` splits one pass over the data into several (sub)epochs,
``repeat_epoch`` repeats, ``_num_shards`` / ``_shard_index`` split further across ranks. Without sharding, distributed
ranks de-correlate by ``random_seed_offset = rank * 16127``.

Parity: returnn/datasets/basic.py (Dataset :39, get_seq_order_for_epoch :508-681, _apply_partition_epoch_and_sharding
:684-714, _get_default_random_seed_offset :267-293, DatasetSeq :1424, init_dataset :1536, generate_batches :1266-1409).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple, Union
import functools
import math
import os
import sys
import numpy
from ..utils.basic import NumbersDict, OptionalNotImplementedError, get_fwd_compat_kwargs
from ..log import log

__all__ = ["Dataset", "DatasetSeq", "init_dataset", "init_dataset_via_str", "get_dataset_class", "set_config_extern_data_from_dataset",
           "convert_data_dims", "shapes_for_batches"]


class Dataset:
    """
    Base class. Subclasses implement ``init_seq_order``, ``_load_seqs`` (or the streaming API of
    :class:`returnn_b200.datasets.cached2.CachedDataset2`), ``get_data`` and the metadata.
    """

    def __init__(self, name: Optional[str] = None, window: int = 1, context_window=None, chunking=None,
                 seq_ordering: Union[str, Callable] = "default", fixed_random_seed: Optional[int] = None,
                 random_seed_offset: Optional[int] = None, partition_epoch: Optional[int] = None, repeat_epoch: Optional[int] = None,
                 seq_list_filter_file: Optional[str] = None, unique_seq_tags: bool = False, seq_order_seq_lens_file: Optional[str] = None,
                 shuffle_frames_of_nseqs: int = 0, min_chunk_size=0, chunking_variance: float = 0, estimated_num_seqs: Optional[int] = None,
                 _num_shards: int = 1, _shard_index: int = 0):
        self.name = name or ("dataset_id%s" % id(self))
        self.lock = None
        self.rnn_layer_sizes: List[int] = []
        self.num_inputs = 0
        self.num_outputs: Optional[Dict[str, Tuple[int, int]]] = None
        self.window = window
        self.seq_ordering = seq_ordering
        self.fixed_random_seed = fixed_random_seed
        if random_seed_offset is None:
            random_seed_offset = self._get_default_random_seed_offset()
        self.random_seed_offset = random_seed_offset
        self.partition_epoch = partition_epoch or 1
        self.repeat_epoch = repeat_epoch or 1
        self._seq_list_filter_file = seq_list_filter_file
        self.seq_tags_filter = set(self._load_seq_list_file(seq_list_filter_file)) if seq_list_filter_file else None
        self.unique_seq_tags = unique_seq_tags
        self._seq_order_seq_lens_file = seq_order_seq_lens_file
        self._seq_order_seq_lens_by_idx = None
        self.labels: Dict[str, List[str]] = {}
        self.weights = {}
        self._num_timesteps = 0
        self._num_seqs = 0
        self._estimated_num_seqs = estimated_num_seqs
        self.min_chunk_size = NumbersDict(min_chunk_size)
        self.chunking_variance = chunking_variance
        self._chunking = chunking
        self.chunk_size, self.chunk_step, self.custom_chunking_func = self._parse_chunking(chunking)
        if isinstance(context_window, (tuple, list)):
            assert len(context_window) == 2
            for elem in context_window:
                assert isinstance(elem, dict)
            self.ctx_left = NumbersDict(numbers_dict=context_window[0])
            self.ctx_right = NumbersDict(numbers_dict=context_window[1])
        else:
            if context_window is None:
                context_window = NumbersDict()
            elif isinstance(context_window, int):
                context_window = NumbersDict(numbers_dict={"data": context_window})
            elif isinstance(context_window, dict):
                context_window = NumbersDict(numbers_dict=context_window)
            assert isinstance(context_window, NumbersDict)
            ctx_total = NumbersDict.max([context_window, 1]) - 1
            self.ctx_left = ctx_total // 2
            self.ctx_right = ctx_total - self.ctx_left
        self.shuffle_frames_of_nseqs = shuffle_frames_of_nseqs
        self.epoch: Optional[int] = None
        self.zpad = None
        assert 0 <= _shard_index < _num_shards
        self._num_shards = _num_shards
        self._shard_index = _shard_index

    def __repr__(self):
        return "<%s %r epoch=%s>" % (self.__class__.__name__, getattr(self, "name", "<unknown>"), getattr(self, "epoch", None))

    _getnewargs_exclude_attrs = set()

    @staticmethod
    def _create_from_reduce(cls, kwargs, state) -> "Dataset":
        """pickle helper: re-create from the constructor kwargs, then restore the extra state"""
        ds = cls(**kwargs)
        for attr, value in state.items():
            setattr(ds, attr, value)
        return ds

    def _ctor_kwargs(self) -> Dict[str, Any]:
        """the kwargs this object was created with; recorded by :func:`init_dataset` and by ``__init_subclass__``"""
        return dict(getattr(self, "_init_kwargs", {}))

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        orig_init = cls.__dict__.get("__init__")
        if orig_init is None:
            return

        @functools.wraps(orig_init)
        def wrapped_init(self, *args, **kw):
            if not hasattr(self, "_init_kwargs"):
                import inspect

                try:
                    bound = inspect.signature(orig_init).bind(self, *args, **kw)
                    d = {}
                    for k, v in list(bound.arguments.items())[1:]:
                        p = inspect.signature(orig_init).parameters[k]
                        if p.kind == inspect.Parameter.VAR_KEYWORD:
                            d.update(v)
                        elif p.kind == inspect.Parameter.VAR_POSITIONAL:
                            raise TypeError("positional varargs")
                        else:
                            d[k] = v
                    object.__setattr__(self, "_init_kwargs", d)
                except TypeError:
                    object.__setattr__(self, "_init_kwargs", None)
            orig_init(self, *args, **kw)

        cls.__init__ = wrapped_init

    def __reduce__(self):
        kwargs = getattr(self, "_init_kwargs", None)
        if kwargs is None:
            raise TypeError("%r cannot be pickled: constructor args unknown" % self)
        state = {attr: getattr(self, attr) for attr in ["epoch", "zpad"]}
        return Dataset._create_from_reduce, (self.__class__, kwargs, state)

    @staticmethod
    def _get_default_random_seed_offset() -> int:
        """under distributed training every rank gets another offset, so that ranks see different orders"""
        from ..config import get_global_config

        config = get_global_config(raise_exception=False)
        if not config:
            return 0
        if config.typed_value("torch_distributed") is not None:
            from ..torch import distributed as _dist

            ctx = _dist.get_ctx(config=config)
            if ctx is not None:
                return ctx.rank() * 16127
        env = os.environ.get("RANK")
        if config.is_true("use_horovod") and env is not None:
            return int(env) * 16127
        return 0

    @staticmethod
    def _parse_chunking(chunking):
        """:return: chunk_size, chunk_step, custom_chunking_func"""
        if callable(chunking):
            return None, None, chunking
        if isinstance(chunking, str):
            if ":" in chunking:
                chunking = tuple(map(int, chunking.split(":")))
            else:
                chunking = int(chunking)
        if not isinstance(chunking, (tuple, list)):
            chunking = (chunking, None)
        chunk_size, chunk_step = chunking
        if chunk_size is None:
            chunk_size = 0
        assert isinstance(chunk_size, (int, dict, NumbersDict))
        chunk_size = NumbersDict(chunk_size)
        assert chunk_size.min_value() >= 0
        if chunk_step in (None, 0):
            chunk_step = chunk_size
        assert isinstance(chunk_step, (int, dict, NumbersDict))
        chunk_step = NumbersDict(chunk_step)
        if chunk_size != 0:
            assert sorted(chunk_step.keys()) == sorted(chunk_size.keys())
            assert chunk_step.max_value() > 0, "chunking step must be positive (for some key)"
        return chunk_size, chunk_step, None

    @staticmethod
    def _load_seq_list_file(filename: str, use_cache_manager: bool = False, expect_list: bool = True):
        """text (one tag per line), .gz, or pickle"""
        if filename.endswith(".pkl"):
            import pickle

            return pickle.load(open(filename, "rb"))
        if filename.endswith(".gz"):
            import gzip

            return gzip.open(filename, "rt").read().splitlines()
        return open(filename).read().splitlines()

    # -- sequence order ----------------------------------------------------------------------------
    def is_cached(self, start: int, end: int) -> bool:
        """whether [start, end) is in memory"""
        return False

    def get_seq_length(self, seq_idx: int) -> NumbersDict:
        """lengths per data key"""
        return NumbersDict({k: self.get_data(seq_idx, k).shape[0] for k in self.get_data_keys()})

    def get_estimated_seq_length(self, seq_idx: int) -> int:
        """in case the real length is expensive"""
        raise OptionalNotImplementedError

    def get_num_timesteps(self) -> int:
        """total frames"""
        assert self._num_timesteps > 0
        return self._num_timesteps

    def load_seqs(self, start: int, end: int):
        """make [start, end) available for get_data"""
        assert start >= 0
        assert start <= end
        if self.is_cached(start, end):
            return
        if self.shuffle_frames_of_nseqs > 0:
            start, end = self._get_shuffle_frames_range(start, end)
        self._load_seqs(start, end)

    def _sliding_window(self, xr: numpy.ndarray) -> numpy.ndarray:
        """
        :param xr: [time, feature]
        :return: [time, window * feature]: frame t is the concatenation of frames t - window//2 .. t + window//2, zeros outside
        """
        half = int(self.window) // 2
        t, f = xr.shape
        padded = numpy.concatenate([numpy.zeros((half, f), dtype=xr.dtype), xr, numpy.zeros((half, f), dtype=xr.dtype)], axis=0)
        view = numpy.lib.stride_tricks.sliding_window_view(padded, (2 * half + 1, f))[:, 0]  # [time, window, feature]
        return numpy.ascontiguousarray(view.reshape(t, (2 * half + 1) * f))

    def _get_shuffle_frames_range(self, start, end):
        n = self.shuffle_frames_of_nseqs
        return start - start % n, end + (n - end % n) % n

    def _load_seqs(self, start: int, end: int):
        raise NotImplementedError

    def _get_seq_order_seq_lens_by_idx(self, seq_idx: int):
        if self._seq_order_seq_lens_by_idx is None:
            assert self._seq_order_seq_lens_file
            content = self._load_seq_list_file(self._seq_order_seq_lens_file, expect_list=False) if self._seq_order_seq_lens_file.endswith(".pkl") else eval(
                (lambda f: __import__("gzip").open(f, "rt").read() if f.endswith(".gz") else open(f).read())(self._seq_order_seq_lens_file))
            all_tags = self.get_all_tags()
            self._seq_order_seq_lens_by_idx = [content[t] for t in all_tags]
        return self._seq_order_seq_lens_by_idx[seq_idx]

    def _get_random_seed_for_epoch(self, epoch: Optional[int], num_epochs_fixed: int = 1) -> int:
        if self.fixed_random_seed is not None:
            return self.fixed_random_seed
        seed = epoch or 1
        if self.partition_epoch > 1:
            seed = (seed - 1) // self.partition_epoch + 1
        if num_epochs_fixed > 1:
            seed = (seed - 1) // num_epochs_fixed + 1
        return seed + self.random_seed_offset

    def get_seq_order_for_epoch(self, epoch: Optional[int], num_seqs: int,
                                get_seq_len: Optional[Callable[[int], Union[int, float]]] = None) -> Sequence[int]:
        """
        :return: order for the epoch: position -> underlying sequence index
        """
        if epoch is None:
            return []
        assert num_seqs > 0 and num_seqs == int(num_seqs)
        num_seqs = int(num_seqs)
        if self._seq_order_seq_lens_file:
            get_seq_len = self._get_seq_order_seq_lens_by_idx
        method = self.seq_ordering
        if callable(method):
            method = method(epoch=epoch, **get_fwd_compat_kwargs())
            if not isinstance(method, str):
                raise TypeError("seq_ordering function should return a str, got %r" % (method,))
        elif not isinstance(method, str):
            raise TypeError("seq_ordering %r: unexpected type" % (method,))
        name, _, arg_str = method.partition(":")
        args = arg_str.split(":") if arg_str else []

        def lens_array():
            assert get_seq_len, "seq_ordering %r needs sequence lengths" % method
            return numpy.array([get_seq_len(i) for i in range(num_seqs)])

        def bins_and_nth():
            bins = 2
            if args:
                bins = max(num_seqs // int(args[0][1:]), 2) if args[0].startswith(".") else int(args[0])
            nth = int(args[1]) if len(args) > 1 else 1
            return bins, nth

        if name == "default":
            seq_index: Any = range(num_seqs)
        elif name == "default_every_n":
            num = int(args[0])
            seq_index = numpy.arange(num_seqs // num, dtype="int64").repeat(num)
            for i in range(1, num):
                seq_index[i::num] += i * (num_seqs // num)
        elif name == "reverse":
            seq_index = range(num_seqs - 1, -1, -1)
        elif name in ("sorted", "sorted_reverse"):
            lens = lens_array()
            seq_index = numpy.argsort(-lens if name == "sorted_reverse" else lens, kind="stable")
        elif name == "random":
            rng = numpy.random.RandomState(self._get_random_seed_for_epoch(epoch, int(args[0]) if args else 1))
            seq_index = rng.permutation(num_seqs)
        elif name == "random_sample":
            rng = numpy.random.RandomState(self._get_random_seed_for_epoch(epoch, int(args[0]) if args else 1))
            seq_index = rng.randint(0, num_seqs, size=num_seqs)
        elif name in ("sort_bin_shuffle", "sort_bin_shuffle_x2"):
            assert get_seq_len
            bins, nth = bins_and_nth()
            rng = numpy.random.RandomState(self._get_random_seed_for_epoch(epoch, nth))
            perm = rng.permutation(num_seqs).tolist()
            perm.sort(key=get_seq_len)
            parts = []
            for i in rng.permutation(bins):
                lo = i * len(perm) // bins
                hi = len(perm) if i == bins - 1 else (i + 1) * len(perm) // bins
                part = perm[lo:hi]
                if name == "sort_bin_shuffle_x2":
                    rng.shuffle(part)
                parts.append(part)
            seq_index = numpy.concatenate(parts)
        elif name == "laplace":
            bins, nth = bins_and_nth()
            lens = lens_array()
            rng = numpy.random.RandomState(self._get_random_seed_for_epoch(epoch, nth))
            perm = rng.permutation(num_seqs)
            parts = []
            for i in range(bins):
                part = perm[i * len(perm) // bins: (i + 1) * len(perm) // bins]
                key = lens[part]
                parts.append(part[numpy.argsort(-key if i % 2 == 1 else key, kind="stable")])
            seq_index = numpy.concatenate(parts)
        else:
            raise ValueError("invalid seq_ordering %r" % (method,))
        if self.unique_seq_tags:
            tags = self.get_all_tags()
            seen = set()
            uniq = []
            for i in seq_index:
                if tags[i] not in seen:
                    seen.add(tags[i])
                    uniq.append(i)
            seq_index = uniq
        if self.partition_epoch > 1 or self._num_shards > 1:
            seq_index = self._apply_partition_epoch_and_sharding(seq_index, self.partition_epoch, epoch, self._num_shards, self._shard_index)
        if self.repeat_epoch > 1:
            seq_index = list(seq_index) * self.repeat_epoch
        if self.seq_tags_filter is not None:
            assert len(seq_index)
            tags = self.get_all_tags()
            assert len(tags) == num_seqs == self.get_total_num_seqs()
            old = seq_index
            seq_index = [i for i in seq_index if tags[i] in self.seq_tags_filter]
            assert seq_index, "%s: empty after applying seq_list_filter_file. Example filter tags: %r, used tags: %r" % (
                self, sorted(self.seq_tags_filter)[:3], [tags[i] for i in old[:3]])
        return seq_index

    @classmethod
    def _apply_partition_epoch_and_sharding(cls, seq_index: Sequence[int], partition_epoch: int, epoch: Optional[int],
                                            num_shards: int, shard_index: int) -> Sequence[int]:
        """contiguous slice ``((epoch-1) % partition_epoch) * num_shards + shard_index`` of ``partition_epoch * num_shards`` near-equal parts"""
        assert 0 <= shard_index < num_shards
        n = len(seq_index)
        parts = partition_epoch * num_shards
        cur = (((epoch or 1) - 1) % partition_epoch) * num_shards + shard_index
        base, extra = divmod(n, parts)
        start = cur * base + min(cur, extra)
        size = base + (1 if cur < extra else 0)
        return seq_index[start: start + size]

    def supports_sharding(self) -> bool:
        """whether _num_shards/_shard_index are honoured"""
        return False

    def supports_seq_order_sorting(self) -> bool:
        """whether sorted orders are possible (lengths known up front)"""
        return False

    def init_seq_order(self, epoch: Optional[int] = None, seq_list: Optional[Sequence[str]] = None,
                       seq_order: Optional[Sequence[int]] = None) -> bool:
        """
        Prepare the (sub)epoch.

        :param epoch: None only to "initialise without an epoch" (no data access yet)
        :param seq_list: explicit list of seq tags instead of the ordering
        :param seq_order: explicit list of underlying indices
        :return: whether the order changed
        """
        self.epoch = epoch
        self.rnd_seq_drop = numpy.random.RandomState((epoch or 1) + self.random_seed_offset)
        return False

    def finish_epoch(self, *, free_resources: bool = False):
        """called at the end of the epoch"""
        self.epoch = None

    def get_current_seq_order(self) -> Sequence[int]:
        """the underlying indices of the current order"""
        raise OptionalNotImplementedError

    def _base_init(self):
        self.nbytes = 0
        self.zpad = None
        assert self.num_outputs
        if not self.num_inputs:
            assert not self.window or self.window in (0, 1) or "data" in self.num_outputs
            return
        assert self.num_inputs > 0
        assert self.window > 0
        if int(self.window) % 2 == 0:
            self.window += 1
        self.nbytes = numpy.array([], dtype=numpy.float32).itemsize * (self.num_inputs * self.window + 1 + 1)
        if self.window > 1:
            self.zpad = numpy.zeros((int(self.window) // 2, self.num_inputs), dtype=numpy.float32)

    def initialize(self):
        """after construction: base init + first (epoch-less) seq order"""
        self._base_init()
        self.init_seq_order()

    # -- data access --------------------------------------------------------------------------------
    def get_data(self, seq_idx: int, key: str) -> numpy.ndarray:
        """array [T, ...] of the (loaded) sequence"""
        raise NotImplementedError

    def get_input_data(self, seq_idx: int) -> numpy.ndarray:
        """get_data(seq_idx, "data")"""
        return self.get_data(seq_idx, "data")

    def get_targets(self, target: str, seq_idx: int) -> numpy.ndarray:
        """get_data(seq_idx, target)"""
        return self.get_data(seq_idx, target)

    def get_data_slice(self, seq_idx: int, key: str, start_frame: int, end_frame: int) -> numpy.ndarray:
        """frames [start, end) with context-window zero padding"""
        if "[sparse:" in key and (start_frame > 0 or end_frame < self.get_seq_length(seq_idx)[key]):
            return self._get_data_slice_sparse(seq_idx, key, start_frame, end_frame)
        data = self.get_data(seq_idx, key)
        return data[start_frame:end_frame]

    def _get_data_slice_sparse(self, seq_idx, key, start_frame, end_frame):
        raise NotImplementedError("sparse COO slicing")

    def get_tag(self, sorted_seq_idx: int) -> str:
        """unique name of the sequence"""
        return "seq-%i" % sorted_seq_idx

    def get_all_tags(self) -> List[str]:
        """all tags, in underlying (unsorted) order"""
        raise OptionalNotImplementedError("%s get_all_tags not implemented" % self)

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        """number of seqs over a whole pass, independent of partition_epoch"""
        raise OptionalNotImplementedError("%s get_total_num_seqs not implemented" % self)

    def have_corpus_seq_idx(self) -> bool:
        """whether get_corpus_seq_idx works"""
        return False

    def get_corpus_seq_idx(self, seq_idx: int) -> int:
        """sorted idx -> underlying idx"""
        if self.seq_ordering == "default" and self.partition_epoch == 1:
            return seq_idx
        raise OptionalNotImplementedError

    def have_get_corpus_seq(self) -> bool:
        """whether get_corpus_seq works (random access by underlying idx)"""
        return False

    def get_corpus_seq(self, corpus_seq_idx: int) -> "DatasetSeq":
        """random access"""
        raise OptionalNotImplementedError

    def has_ctc_targets(self) -> bool:
        """legacy"""
        return False

    def get_max_ctc_length(self) -> int:
        """legacy"""
        return 0

    @classmethod
    def generic_complete_frac(cls, seq_idx: int, num_seqs: Optional[int]) -> float:
        """fraction in [0,1]; with unknown num_seqs an asymptotic guess"""
        if num_seqs:
            return min(float(seq_idx + 1) / num_seqs, 1.0)
        return 1.0 - math.exp(-seq_idx / 10000.0) if seq_idx else 0.0

    def get_complete_frac(self, sorted_seq_idx: int, *, allow_only_lr_suitable: bool = False, **kwargs) -> Optional[float]:
        """how far through the epoch seq_idx is"""
        try:
            num_seqs = self.num_seqs
        except Exception:
            try:
                num_seqs = self.estimated_num_seqs
                if allow_only_lr_suitable:
                    return None
            except Exception:
                num_seqs = None
                if allow_only_lr_suitable:
                    return None
        return self.generic_complete_frac(sorted_seq_idx, num_seqs)

    @property
    def num_seqs(self) -> int:
        """number of sequences in this (sub)epoch"""
        raise NotImplementedError

    @property
    def estimated_num_seqs(self) -> Optional[int]:
        """estimate if exact is unknown"""
        try:
            return self.num_seqs
        except Exception:
            pass
        if self._estimated_num_seqs is not None:
            return self._estimated_num_seqs
        return None

    def get_data_keys(self) -> List[str]:
        """all data keys, "data" first"""
        return ["data"] + self.get_target_list()

    def get_target_list(self) -> List[str]:
        """keys which are targets"""
        return ["classes"]

    def get_data_dim(self, key: str) -> int:
        """feature dim or number of classes"""
        if key == "data" and key not in (self.num_outputs or {}):
            return self.num_inputs * self.window
        return self.num_outputs[key][0]

    def get_data_dtype(self, key: str) -> str:
        """numpy dtype name"""
        if self.is_data_sparse(key):
            return "int32"
        return "float32"

    def is_data_sparse(self, key: str) -> bool:
        """class indices"""
        if key in (self.num_outputs or {}):
            return self.num_outputs[key][1] <= 1
        if key == "data":
            return False
        return True

    def get_data_shape(self, key: str) -> List[int]:
        """shape without the time axis"""
        if self.is_data_sparse(key):
            return []
        return [self.get_data_dim(key)]

    def get_extern_data(self):
        """extern_data template dict from the dataset metadata"""
        from ..tensor import Dim, batch_dim

        res = {}
        for key in self.get_data_keys():
            dim = self.get_data_dim(key)
            ndim = self.num_outputs[key][1] if key in (self.num_outputs or {}) else 2
            time_dim = Dim(None, name="%s:time" % key, kind=Dim.Types.Spatial)
            if self.is_data_sparse(key):
                sparse_dim = Dim(dim, name="%s:classes" % key, kind=Dim.Types.Feature)
                if key in self.labels and len(self.labels[key]) == dim:
                    from .util.vocabulary import Vocabulary

                    sparse_dim.vocab = Vocabulary.create_vocab_from_labels(self.labels[key])
                dims = [batch_dim] + ([time_dim] if ndim >= 1 else [])
                res[key] = {"dims": dims, "sparse_dim": sparse_dim, "dtype": self.get_data_dtype(key)}
            else:
                shape = self.get_data_shape(key)
                dims = [batch_dim, time_dim] + [Dim(s, name="%s:feature%i" % (key, i), kind=Dim.Types.Feature) for i, s in enumerate(shape)]
                res[key] = {"dims": dims, "dtype": self.get_data_dtype(key)}
        return res

    def is_less_than_num_seqs(self, n: int) -> bool:
        """n < num_seqs (subclasses with unknown num_seqs override)"""
        return n < self.num_seqs

    def can_serialize_data(self, key: str) -> bool:
        """whether serialize_data works"""
        return key in self.labels

    def serialize_data(self, key: str, data: numpy.ndarray) -> str:
        """labels as text"""
        labels = self.labels[key]
        if len(labels) < 1000 and all(len(lb) == 1 for lb in labels):
            return "".join(labels[int(i)] for i in data)
        return " ".join(labels[int(i)] for i in data)

    # -- chunking / legacy batching -----------------------------------------------------------------
    def iterate_seqs(self, recurrent_net: bool = True, used_data_keys=None) -> Iterator[Tuple[int, NumbersDict, NumbersDict]]:
        """
        Yield (seq_idx, chunk_start, chunk_end) over all sequences, applying chunking.
        """
        if self.custom_chunking_func:
            sentinel = object()
            yield from self.custom_chunking_func(dataset=self, seq_idx_start=0, recurrent_net=recurrent_net,
                                                 used_data_keys=used_data_keys, **get_fwd_compat_kwargs())
            return
        chunk_size = self.chunk_size
        chunk_step = self.chunk_step
        if not recurrent_net and chunk_size != 0:
            chunk_size = NumbersDict(0)
        s = 0
        while self.is_less_than_num_seqs(s):
            length = self.get_seq_length(s)
            if used_data_keys is not None:
                length = NumbersDict({k: length[k] for k in used_data_keys if k in length.dict})
            if chunk_size == 0:
                yield s, NumbersDict.constant_like(0, numbers_dict=length), length
            else:
                default_key = "data" if "data" in length.dict else sorted(length.keys())[0]
                chunk_size_orig = chunk_size.copy()
                chunk_step_orig = chunk_step.copy()
                cs, cst = chunk_size, chunk_step
                if self.chunking_variance > 0:
                    var = 1.0 - self.rnd_seq_drop.random_sample() * self.chunking_variance
                    for k in list(cs.keys()):
                        cs[k] = max(int(cs[k] * var), 1)
                        cst[k] = max(int(cst[k] * var), 1)
                t = NumbersDict.constant_like(0, numbers_dict=length)
                keys_with_full_seqs = [k for k in length.keys() if cs.get(k, cs.value if cs.value is not None else 0) == 0]
                limit = length[default_key]
                while t[default_key] < limit:
                    chunk_start = t.copy()
                    chunk_end = NumbersDict.min([t + cs, length])
                    for k in keys_with_full_seqs:
                        chunk_start[k] = 0
                        chunk_end[k] = length[k]
                    if length.value is None:
                        chunk_start.value = None
                        chunk_end.value = None
                    yield s, chunk_start, chunk_end
                    t += cst
                    if length[default_key] - t[default_key] <= self.min_chunk_size.get(default_key, self.min_chunk_size.value or 0):
                        break
                chunk_size, chunk_step = chunk_size_orig, chunk_step_orig
            s += 1

    def get_start_end_frames_full_seq(self, seq_idx: int) -> Tuple[NumbersDict, NumbersDict]:
        """(0, length)"""
        end = self.get_seq_length(seq_idx)
        return NumbersDict.constant_like(0, numbers_dict=end), end

    def sample(self, seq_idx: int) -> bool:
        """legacy seq weights"""
        return True

    def generate_batches(self, recurrent_net: bool = True, batch_size=0, max_seqs: int = -1, max_seq_length=sys.maxsize,
                         max_pad_size=None, min_seq_length=0, pruning: float = 0.0, seq_drop: float = 0.0,
                         max_total_num_seqs: int = -1, used_data_keys=None):
        """
        Legacy in-dataset batching: :class:`returnn_b200.engine.batch.BatchSetGenerator` over all (chunked) sequences.
        """
        from ..engine.batch import BatchSetGenerator

        return BatchSetGenerator(self, self._generate_batches(
            recurrent_net=recurrent_net, batch_size=batch_size, max_seqs=max_seqs, max_seq_length=max_seq_length,
            max_pad_size=max_pad_size, min_seq_length=min_seq_length, seq_drop=seq_drop, max_total_num_seqs=max_total_num_seqs,
            used_data_keys=used_data_keys))

    def _generate_batches(self, recurrent_net, batch_size, max_seqs=-1, max_seq_length=sys.maxsize, max_pad_size=None,
                          min_seq_length=0, seq_drop=0.0, max_total_num_seqs=-1, used_data_keys=None):
        from ..engine.batch import Batch

        if not batch_size:
            batch_size = sys.maxsize
        batch_size = NumbersDict(batch_size)
        assert not batch_size.any_compare(NumbersDict(0), (lambda a, b: a <= b))
        if max_seqs == -1:
            max_seqs = float("inf")
        if not max_pad_size:
            max_pad_size = None
        max_seq_length = NumbersDict(max_seq_length) if not isinstance(max_seq_length, NumbersDict) else max_seq_length
        min_seq_length = NumbersDict(min_seq_length) if not isinstance(min_seq_length, NumbersDict) else min_seq_length
        batch = Batch()
        total_num_seqs = 0
        last_seq_idx = -1
        for seq_idx, t_start, t_end in self.iterate_seqs(recurrent_net=recurrent_net, used_data_keys=used_data_keys):
            if not self.sample(seq_idx):
                continue
            if total_num_seqs > max_total_num_seqs >= 0:
                break
            length = t_end - t_start
            if length.any_compare(max_seq_length, (lambda a, b: a > b)):
                continue
            if length.any_compare(min_seq_length, (lambda a, b: a < b)):
                continue
            if length.max_value() > batch_size.max_value():
                print("warning: sequence length (%i) larger than limit (%i)" % (length.max_value(), batch_size.max_value()), file=log.v4)
            if self.rnd_seq_drop.random_sample() < seq_drop:
                continue
            dt, ds = batch.try_sequence_as_slice(length)
            if batch.num_slices >= 1:
                if (dt * ds).any_compare(batch_size, (lambda a, b: a > b)):
                    yield batch
                    batch = Batch()
                elif ds > max_seqs:
                    yield batch
                    batch = Batch()
                elif max_pad_size is not None and (dt * ds - batch.get_total_num_frames() - length).max_value() > max_pad_size:
                    yield batch
                    batch = Batch()
            batch.add_sequence_as_slice(seq_idx=seq_idx, seq_start_frame=t_start, length=length)
            if seq_idx != last_seq_idx:
                last_seq_idx = seq_idx
                total_num_seqs += 1
        if batch.get_all_slices_num_frames().max_value() > 0:
            yield batch

    @classmethod
    def index_shape_for_batches(cls, batches, data_key="data"):
        """[max time, num slices] for a list of batches"""
        shape = [0, 0]
        for batch in batches:
            shape = [max(shape[0], batch.max_num_frames_per_slice[data_key]), shape[1] + batch.num_slices]
        return shape


class DatasetSeq:
    """one sequence: features dict, tag, index"""

    def __init__(self, seq_idx: int, features, targets=None, seq_tag: Optional[str] = None):
        """
        :param features: array (key "data") or dict key -> array
        :param targets: array (key "classes") or dict, merged into features
        """
        assert isinstance(seq_idx, (int, numpy.integer))
        self.seq_idx = int(seq_idx)
        self.seq_tag = seq_tag or ("seq-%i" % seq_idx)
        if not isinstance(features, dict):
            assert isinstance(features, numpy.ndarray)
            features = {"data": features}
            if targets is None:
                targets = {}
            if isinstance(targets, numpy.ndarray):
                targets = {"classes": targets}
            assert isinstance(targets, dict)
            features.update(targets)
            targets = None
        assert isinstance(features, dict) and targets is None
        for v in features.values():
            assert isinstance(v, numpy.ndarray)
        self.features = features

    @property
    def num_frames(self) -> NumbersDict:
        """lengths per key"""
        return NumbersDict({k: (v.shape[0] if v.ndim >= 1 else 1) for k, v in self.features.items()})

    def get_data(self, key: str) -> numpy.ndarray:
        """array for key"""
        return self.features[key]

    def get_data_keys(self):
        """keys"""
        return self.features.keys()

    def __repr__(self):
        return "<DataCache seq_idx=%i>" % self.seq_idx


_dataset_classes: Dict[str, type] = {}


def _dataset_modules() -> List[str]:
    here = os.path.dirname(os.path.abspath(__file__))
    mods = []
    for f in sorted(os.listdir(here)):
        if f.endswith(".py") and not f.startswith("_"):
            mods.append(f[:-3])
    return mods


def get_dataset_class(name: Union[str, type]) -> Optional[type]:
    """class by name over all dataset modules"""
    if isinstance(name, type):
        return name
    if name in _dataset_classes:
        return _dataset_classes[name]
    import importlib

    if "." in name:
        mod_name, cls_name = name.rsplit(".", 1)
        if mod_name.startswith("returnn."):
            mod_name = "returnn_b200." + mod_name[len("returnn."):]
        mod = importlib.import_module(mod_name)
        return getattr(mod, cls_name)
    for mod_name in _dataset_modules():
        try:
            mod = importlib.import_module("returnn_b200.datasets." + mod_name)
        except ImportError:
            continue
        for k, v in vars(mod).items():
            if isinstance(v, type) and issubclass(v, Dataset):
                _dataset_classes.setdefault(k, v)
    return _dataset_classes.get(name)


def init_dataset(kwargs: Union[Dict[str, Any], str, Callable, Dataset], extra_kwargs: Optional[Dict[str, Any]] = None,
                 default_kwargs: Optional[Dict[str, Any]] = None, parent_dataset: Optional[Dataset] = None) -> Dataset:
    """
    :param kwargs: ``{"class": "<ClassName>", ...}``, a callable returning that, a Dataset, or a legacy string
    """
    assert kwargs
    if isinstance(kwargs, Dataset):
        data = kwargs
        data.initialize()
        return data
    if callable(kwargs):
        return init_dataset(kwargs(), extra_kwargs=extra_kwargs, default_kwargs=default_kwargs)
    if isinstance(kwargs, str):
        if kwargs.startswith("{"):
            kwargs = eval(kwargs)
        elif kwargs.startswith("config:"):
            from ..config import get_global_config

            config = get_global_config()
            data = eval(kwargs[len("config:"):], config.typed_dict, config.typed_dict)
            return init_dataset(data, extra_kwargs=extra_kwargs, default_kwargs=default_kwargs)
        else:
            config_str = kwargs
            kwargs = {}
            if default_kwargs:
                kwargs.update(default_kwargs)
            if extra_kwargs:
                kwargs.update(extra_kwargs)
            return init_dataset_via_str(config_str=config_str, **kwargs)
    assert isinstance(kwargs, dict)
    kwargs = kwargs.copy()
    assert "class" in kwargs, "dataset dict needs a 'class': %r" % (kwargs,)
    clazz_name = kwargs.pop("class")
    clazz = get_dataset_class(clazz_name)
    if not clazz:
        raise Exception("Dataset class %r not found" % clazz_name)
    if default_kwargs:
        for k, v in default_kwargs.items():
            kwargs.setdefault(k, v)
    if extra_kwargs:
        kwargs.update(extra_kwargs)
    if parent_dataset is not None and "random_seed_offset" not in kwargs:
        kwargs["random_seed_offset"] = parent_dataset.random_seed_offset
    obj = clazz(**kwargs)
    assert isinstance(obj, Dataset)
    obj.initialize()
    return obj


def extend_dataset_dict_from_parent_dataset(dataset_dict: Dict[str, Any], parent_dataset: Optional[Dataset]) -> Dict[str, Any]:
    """
    What a wrapping dataset hands down to the dataset it creates: options that must agree between the two (the per-rank seed offset), unless
    the inner description sets them itself. Parity: returnn/datasets/basic.py:1625.

    :return: a copy of ``dataset_dict`` with those options filled in
    """
    res = dict(dataset_dict)
    if parent_dataset is not None and "random_seed_offset" not in res:
        res["random_seed_offset"] = parent_dataset.random_seed_offset
    return res


def init_dataset_via_str(config_str: str, config=None, cache_byte_size=None, **kwargs) -> Dataset:
    """
    Legacy: ``"<Class>:<args>"`` or a comma-separated list of HDF files.
    """
    kwargs = kwargs.copy()
    if "window" not in kwargs and config:
        kwargs["window"] = config.int("window", 1)
    if config:
        for k in ("chunking", "min_chunk_size", "chunking_variance", "batching"):
            if k == "batching":
                if "seq_ordering" not in kwargs and config.has("batching"):
                    kwargs["seq_ordering"] = config.value("batching", "default")
            elif k not in kwargs and config.has(k):
                kwargs[k] = config.typed_value(k) if config.is_typed(k) else config.value(k, None)
    if ":" in config_str and not config_str.startswith("/") and not os.path.exists(config_str.split(",")[0]):
        cls_name, _, args = config_str.partition(":")
        clazz = get_dataset_class(cls_name)
        if clazz is None:
            raise Exception("dataset class %r not found" % cls_name)
        if args.startswith("{"):
            kw = eval(args)
        else:
            kw = {}
            pos = []
            for a in args.split(":") if args else []:
                if "=" in a:
                    k, v = a.split("=", 1)
                    try:
                        kw[k] = eval(v)
                    except Exception:
                        kw[k] = v
                else:
                    try:
                        pos.append(eval(a))
                    except Exception:
                        pos.append(a)
            if pos:
                import inspect

                names = [p for p in inspect.signature(clazz.__init__).parameters][1:]
                for n, v in zip(names, pos):
                    kw[n] = v
        kw.update(kwargs)
        data = clazz(**kw)
    else:
        from .hdf import HDFDataset

        files = config_str.split(",") if config_str else []
        data = HDFDataset(files=files, cache_byte_size=cache_byte_size or 0, **kwargs)
    data.initialize()
    return data


def convert_data_dims(data_dims, leave_dict_as_is: bool = False) -> Dict[str, Any]:
    """``{key: dim | (dim, ndim) | dict}`` -> ``{key: (dim, ndim)}`` or the extern_data dict form"""
    assert isinstance(data_dims, dict)
    res = {}
    for k, v in data_dims.items():
        if isinstance(v, int):
            v = (v, 2 if k == "data" else 1)
        elif isinstance(v, dict):
            if leave_dict_as_is:
                res[k] = v
                continue
            dim = v.get("dim")
            ndim = len(v["shape"]) if "shape" in v else (1 if v.get("sparse") else 2)
            v = (dim, ndim)
        assert isinstance(v, (tuple, list)) and len(v) == 2
        res[k] = tuple(v)
    return res


def shapes_for_batches(batches, data_keys, dataset=None, extern_data=None, enforce_min_len1: bool = False):
    """shape [B, T, ...] per key for a list of legacy batches"""
    assert dataset or extern_data
    all_dims = {}
    for batch in batches:
        for k in data_keys:
            all_dims[k] = max(all_dims.get(k, 0), batch.max_num_frames_per_slice[k])
    n = sum(b.num_slices for b in batches)
    shapes = {}
    for k in data_keys:
        t = max(all_dims.get(k, 0), 1) if enforce_min_len1 else all_dims.get(k, 0)
        shape = [n, t]
        if dataset is not None:
            shape += dataset.get_data_shape(k)
        shapes[k] = shape
    return shapes


def set_config_extern_data_from_dataset(config, dataset: Dataset):
    """set ``extern_data`` in the config from the dataset metadata (when the user did not give it)"""
    config.set("extern_data", dataset.get_extern_data())
