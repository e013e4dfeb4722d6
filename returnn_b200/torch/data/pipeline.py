"""
Data pipeline between a dataset and the train step: length filter, chunking, token-budget batching, optional bucket
batching, batch shuffling, collation (padded or packed), and a DataLoader with non-daemonic spawn workers.

Batching rule (greedy, in order): a batch is flushed when adding the next sequence would make
``(n + 1) * max_len`` exceed ``batch_size`` for any key, or ``n >= max_seqs``, or the unpadded sum exceed
``packed_batch_size``.

Parity: returnn/torch/data/pipeline.py (collate_batch :58-105, ChunkingIterDataPipe :108-192, BatchingIterDataPipe
:224-374, BucketOrderingIterDataPipe :377-470, LenFilterDataPipe :515-552, ShufflingDataPipe :558-674,
create_data_loader_from_batches :677-733, get_batching_iterable_dataset_from_config :473-512).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union
import bisect
import sys
import numpy
import torch
import torch.utils.data
from ...utils.basic import NumbersDict, get_fwd_compat_kwargs

InputType = Union[numpy.ndarray, int, str, float, bool]
OutputType = Union[torch.Tensor, int, str, float, bool, numpy.ndarray]


def create_tensor(array: numpy.ndarray) -> Union[torch.Tensor, numpy.ndarray]:
    """numpy -> torch; string arrays stay numpy"""
    if isinstance(array, torch.Tensor):
        return array
    array = numpy.asarray(array)
    if array.dtype.kind in "UO":
        return array
    if array.dtype == numpy.uint32:
        array = array.astype(numpy.int64)
    if array.ndim > 0 and not array.flags.c_contiguous:
        array = numpy.ascontiguousarray(array)
    return torch.from_numpy(array) if array.flags.writeable else torch.from_numpy(array.copy())


def collate_batch(batch: List[Dict[str, numpy.ndarray]], *, packing: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """
    Merge samples into one tensor per key: padded ``[B, T_max, ...]`` with ``"<key>:seq_len"`` int32 ``[B]``;
    with ``packing`` the sequences of the listed keys are concatenated to ``[sum(T), ...]`` without padding
    (``"<key>:packed"`` = True marks them).
    """
    assert isinstance(batch, list) and batch and isinstance(batch[0], dict)
    res: Dict[str, Any] = {}
    for key in batch[0].keys():
        if key in ("num_seqs", "epoch"):
            res[key] = batch[0][key]
            continue
        if key == "complete_frac":
            res[key] = max(sample[key] for sample in batch)
            continue
        ls = [create_tensor(sample[key]) for sample in batch]
        if isinstance(ls[0], torch.Tensor):
            if ls[0].ndim > 0:
                if packing is not None and (packing.get("keys") is None or key in packing["keys"]):
                    res[key] = torch.cat(ls, dim=0)
                    res["%s:packed" % key] = True
                else:
                    res[key] = torch.nn.utils.rnn.pad_sequence(ls, batch_first=True, padding_value=0)
                res["%s:seq_len" % key] = torch.tensor([v.shape[0] for v in ls], dtype=torch.int32)
            else:
                res[key] = torch.stack(ls, dim=0)
        else:
            res[key] = numpy.stack(ls, axis=0)
    return res


class ChunkingIterDataPipe(torch.utils.data.IterableDataset):
    """splits sequences into chunks ``(size, step)``, per key or for all keys"""

    def __init__(self, dataset: torch.utils.data.IterableDataset, chunking, *, min_chunk_size=0):
        super().__init__()
        from ...datasets.basic import Dataset as _DS

        self._dataset = dataset
        self._chunk_size, self._chunk_step, custom = _DS._parse_chunking(chunking)
        self._min_chunk_size = NumbersDict(min_chunk_size)
        assert not custom, "custom chunking functions are not supported here"

    def __iter__(self) -> Iterable[List[Dict[str, InputType]]]:
        chunking_data_keys = None
        for data_dict in self._dataset:
            if not chunking_data_keys:
                data_keys = [k for k, v in data_dict.items() if isinstance(v, numpy.ndarray) and v.ndim >= 1 and k != "seq_tag"]
                if self._chunk_size.dict:
                    chunking_data_keys = [k for k in data_keys if self._chunk_size.get(k, 0)]
                else:
                    chunking_data_keys = list(data_keys)
                assert chunking_data_keys, "chunking: no data key to chunk"
            # A chunk starts at every multiple of the step inside the sequence (so the tail of a sequence also comes as shorter chunks
            # of its own); chunks shorter than min_chunk_size are left out. All chunked keys must give the same number of chunks.
            pieces: Dict[str, List[numpy.ndarray]] = {}
            n_chunks = None
            for k in chunking_data_keys:
                size, step = self._chunk_size[k], self._chunk_step[k]
                min_size = self._min_chunk_size.get(k, self._min_chunk_size.value or 0)
                v = data_dict[k]
                ks = [v[start: start + size] for start in range(0, len(v), step)]
                ks = [p for p in ks if len(p) >= min_size]
                assert n_chunks is None or n_chunks == len(ks), "chunking: %i chunks for %r, %i for %r" % (len(ks), k, n_chunks, chunking_data_keys[0])
                n_chunks = len(ks)
                pieces[k] = ks
            for c in range(n_chunks or 0):
                chunk = {k: (pieces[k][c] if k in pieces else v) for k, v in data_dict.items()}
                if "seq_tag" in chunk:  # for every sequence, also the ones of a single chunk: all samples of a batch carry the same keys
                    chunk["chunk_idx"] = numpy.array(c, dtype="int32")
                yield chunk

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


class BatchingIterDataPipe(torch.utils.data.IterableDataset):
    """greedy in-order batching under a padded-frames budget"""

    def __init__(self, dataset: torch.utils.data.IterableDataset, batch_size=1, max_seqs=None, packed_batch_size=None):
        super().__init__()
        self._dataset = dataset
        self._max_batch_size = self._parse_batch_size(batch_size)
        self._max_seqs = self._parse_max_seqs(max_seqs)
        self._max_packed_batch_size = self._parse_batch_size(packed_batch_size) if packed_batch_size is not None else None

    @staticmethod
    def _parse_batch_size(batch_size, *, data_dict: Optional[Dict[str, Any]] = None):
        if callable(batch_size):
            if data_dict is None:
                return batch_size
            batch_size = batch_size(**BatchingIterDataPipe._get_user_func_kwargs_from_data_dict(data_dict))
        if isinstance(batch_size, NumbersDict):
            return batch_size
        return NumbersDict(sys.maxsize if (batch_size is None or batch_size == -1 or batch_size == 0) else batch_size)

    @staticmethod
    def _parse_max_seqs(max_seqs, *, data_dict: Optional[Dict[str, Any]] = None):
        if callable(max_seqs):
            if data_dict is None:
                return max_seqs
            max_seqs = max_seqs(**BatchingIterDataPipe._get_user_func_kwargs_from_data_dict(data_dict))
        return sys.maxsize if (max_seqs is None or max_seqs == -1) else max_seqs

    @staticmethod
    def _get_user_func_kwargs_from_data_dict(data_dict: Dict[str, Any]) -> Dict[str, Any]:
        epoch = int(data_dict["epoch"])
        seq_idx = int(data_dict["seq_idx"])
        num_seqs = int(data_dict["num_seqs"])
        complete_frac = float(data_dict["complete_frac"])
        if complete_frac >= 0.0:
            epoch_continuous = epoch - 1 + complete_frac
        elif num_seqs > 0:
            epoch_continuous = epoch - 1 + (seq_idx + 1) / num_seqs
        else:
            epoch_continuous = None
        return {"epoch": epoch, "epoch_continuous": epoch_continuous, "seq_idx": seq_idx, **get_fwd_compat_kwargs()}

    def __iter__(self) -> Iterator[List[Dict[str, numpy.ndarray]]]:
        cur: List[Dict[str, numpy.ndarray]] = []
        cur_max = NumbersDict(0)
        cur_sum = NumbersDict(0)
        for data_dict in self._dataset:
            max_seqs = self._parse_max_seqs(self._max_seqs, data_dict=data_dict)
            max_bs = self._parse_batch_size(self._max_batch_size, data_dict=data_dict)
            max_packed = self._parse_batch_size(self._max_packed_batch_size, data_dict=data_dict) if self._max_packed_batch_size is not None else None
            if len(cur) >= max_seqs:
                yield cur
                cur, cur_max, cur_sum = [], NumbersDict(0), NumbersDict(0)
            lens = NumbersDict({k: v.shape[0] for k, v in data_dict.items() if isinstance(v, numpy.ndarray) and v.shape and v.dtype.kind not in "UO"})
            new_max = NumbersDict.max([cur_max, lens])
            padded = new_max * (len(cur) + 1)
            new_sum = cur_sum + lens
            over = padded.any_compare(max_bs, (lambda a, b: a > b))
            if max_packed is not None:
                over = over or new_sum.any_compare(max_packed, (lambda a, b: a > b))
            if cur and over:
                yield cur
                cur, cur_max, cur_sum = [data_dict], lens, lens
            else:
                cur.append(data_dict)
                cur_max, cur_sum = new_max, new_sum
        if cur:
            yield cur

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


class BucketOrderingIterDataPipe(torch.utils.data.IterableDataset):
    """
    Sequences go into length buckets ``{max_len: max_batch_seqs}``; a bucket is emitted as a batch once full.
    Leftovers are emitted at the end of the epoch.
    """

    def __init__(self, dataset: torch.utils.data.IterableDataset, *, buckets: Sequence[Tuple[int, int]], length_key: str,
                 random_bucket_prob: float = 0.0, seed: Optional[int] = None):
        super().__init__()
        self._dataset = dataset
        self._length_key = length_key
        self._random_bucket_prob = random_bucket_prob
        self._rng = numpy.random.RandomState()
        self._seed = seed % (2 ** 32) if seed is not None else None
        assert buckets, "empty bucket batching configuration"
        if not all(size > 0 and max_seq > 0 for size, max_seq in buckets):
            raise ValueError("bucket sizes and batch sizes must be positive")
        self._max_seq_lens, self._max_bucket_sizes = zip(*sorted(buckets))
        if len(set(self._max_seq_lens)) != len(self._max_seq_lens):
            raise ValueError("seq length buckets must be unique")

    def set_seed(self, seed: int) -> "BucketOrderingIterDataPipe":
        """seed for the random bucket choice"""
        self._seed = seed % (2 ** 32)
        return self

    def __iter__(self):
        if self._seed is not None:
            self._rng.seed(self._seed)
        buckets: List[List[Dict[str, Any]]] = [[] for _ in self._max_bucket_sizes]
        for data_dict in self._dataset:
            n = data_dict[self._length_key].shape[0]
            idx = bisect.bisect_left(self._max_seq_lens, n)
            if idx >= len(self._max_seq_lens):
                raise ValueError("sequence of length %i longer than the largest bucket %i" % (n, self._max_seq_lens[-1]))
            if self._random_bucket_prob > 0.0 and self._rng.rand() < self._random_bucket_prob:
                idx = int(self._rng.randint(idx, len(self._max_bucket_sizes)))
            buckets[idx].append(data_dict)
            if len(buckets[idx]) >= self._max_bucket_sizes[idx]:
                yield buckets[idx]
                buckets[idx] = []
        nonempty = [b for b in buckets if b]
        self._rng.shuffle(nonempty)
        yield from nonempty

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


def balance_batches(batches: List[List[Dict[str, Any]]], *, length_key: str, max_seqs: int = -1,
                    max_padded: Optional[int] = None) -> List[List[Dict[str, Any]]]:
    """
    Redistribute the sequences of ``len(batches)`` consecutive batches so that every batch holds nearly the same number of REAL
    frames (sum of sequence lengths).

    On packed rows the time of a training step follows the real frames of a batch, while the greedy batching rule bounds the
    padded frames: a batch of short sequences holds many more real frames than a batch with one long sequence. In a
    data-parallel job every step then takes as long as the rank with the fullest batch. Longest-first assignment to the currently
    emptiest batch (the LPT rule) evens this out; it is deterministic, so every rank computes the same partition without
    communication. The group as a whole holds the same sequences as before.

    Mixing long and short sequences raises the PADDED size of a batch above what the greedy rule produced (the padded budget
    of a group shrinks when every batch contains a long sequence), so this is for models that compute on packed rows, whose
    memory follows the real frames. ``max_padded`` (optional) bounds ``n * max_len`` per batch; a sequence that fits nowhere
    under it stays in the batch it came from.
    """
    n_bins = len(batches)
    if n_bins <= 1:
        return batches
    items = []
    for b_idx, b in enumerate(batches):
        for s_idx, seq in enumerate(b):
            items.append((int(seq[length_key].shape[0]), b_idx, s_idx))
    items.sort(key=lambda t: (-t[0], t[1], t[2]))
    bins: List[List[Dict[str, Any]]] = [[] for _ in range(n_bins)]
    real = [0] * n_bins
    longest = [0] * n_bins
    leftovers = []
    for length, b_idx, s_idx in items:
        placed = False
        for i in sorted(range(n_bins), key=lambda i: (real[i], i)):
            mx = max(longest[i], length)
            if max_padded is not None and (len(bins[i]) + 1) * mx > max_padded:
                continue
            if max_seqs > 0 and len(bins[i]) >= max_seqs:
                continue
            bins[i].append(batches[b_idx][s_idx])
            real[i] += length
            longest[i] = mx
            placed = True
            break
        if not placed:
            leftovers.append((b_idx, s_idx))
    for b_idx, s_idx in leftovers:
        bins[b_idx].append(batches[b_idx][s_idx])
    return bins


class RankBalancedBatchingIterDataPipe(torch.utils.data.IterableDataset):
    """
    Data-parallel batching with equal work per rank. Every rank reads the SAME sequence stream (same dataset, same seed: set
    ``random_seed_offset`` to 0 on all ranks), forms ``world`` consecutive batches with the usual greedy rule, evens out their real
    frame totals with :func:`balance_batches`, and keeps batch number ``rank`` of every group. A step's batches then differ in
    content but hold the same amount of work on every rank, and no sequence is trained on by two ranks.

    Config: ``torch_batching = {"type": "rank_balanced", "length_key": "data"}`` (rank and world come from the distributed context;
    ``max_padded`` optionally bounds the padded size of a rebalanced batch, see :func:`balance_batches`).
    """

    def __init__(self, dataset: torch.utils.data.IterableDataset, *, batch_size, max_seqs: int = -1, length_key: str = "data",
                 rank: int = 0, world: int = 1, packed_batch_size=None, max_padded: Optional[int] = None):
        super().__init__()
        self._batches = BatchingIterDataPipe(dataset, batch_size=batch_size, max_seqs=max_seqs, packed_batch_size=packed_batch_size)
        self._max_padded = max_padded
        self._max_seqs = max_seqs if max_seqs is not None else -1
        self._length_key = length_key
        self._rank, self._world = rank, world
        assert 0 <= rank < world

    def __iter__(self):
        group: List[List[Dict[str, Any]]] = []
        for batch in self._batches:
            group.append(batch)
            if len(group) == self._world:
                yield balance_batches(group, length_key=self._length_key, max_seqs=self._max_seqs, max_padded=self._max_padded)[self._rank]
                group = []
        # an incomplete last group is dropped on every rank alike: all ranks see the same number of steps

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


def get_batching_iterable_dataset_from_config(*, dataset: torch.utils.data.IterableDataset, config, train: bool) -> torch.utils.data.IterableDataset:
    """batching by config: ``torch_batching`` custom function / dict, else batch_size + max_seqs (+ packed_batch_size)"""
    batch_size = config.typed_value("batch_size", -1)
    batch_size = config.typed_value("batch_size_%s" % ("train" if train else "dev"), batch_size)
    assert batch_size != -1, "batch_size or batch_size_%s not defined in config" % ("train" if train else "dev")
    max_seqs = config.typed_value("max_seqs", -1)
    packed_batch_size = config.typed_value("packed_batch_size", None)
    batches_dataset = None
    custom = config.typed_value("torch_batching", None)
    if isinstance(custom, dict):
        opts = dict(custom)
        kind = opts.pop("type")
        if kind == "bucket":
            batches_dataset = BucketOrderingIterDataPipe(dataset, **opts)
        elif kind == "rank_balanced":
            if "rank" not in opts:
                import torch.distributed as _dist

                opts["rank"] = _dist.get_rank() if _dist.is_available() and _dist.is_initialized() else 0
                opts["world"] = _dist.get_world_size() if _dist.is_available() and _dist.is_initialized() else 1
            batches_dataset = RankBalancedBatchingIterDataPipe(dataset, batch_size=batch_size, max_seqs=max_seqs,
                                                               packed_batch_size=packed_batch_size, **opts)
        else:
            raise ValueError("torch_batching: type must be 'bucket' or 'rank_balanced', got %r" % (kind,))
    elif custom is not None:
        batches_dataset = custom(dataset=dataset, config=config, train=train, **get_fwd_compat_kwargs())
    if batches_dataset is None:
        batches_dataset = BatchingIterDataPipe(dataset, batch_size=batch_size, max_seqs=max_seqs, packed_batch_size=packed_batch_size)
    return batches_dataset


class LenFilterDataPipe(torch.utils.data.IterableDataset):
    """drops sequences outside [min_seq_length, max_seq_length] (per key or for all keys)"""

    def __init__(self, dataset: torch.utils.data.IterableDataset, min_seq_length=None, max_seq_length=None):
        super().__init__()
        self._dataset = dataset
        self._min_seq_length = NumbersDict(0 if min_seq_length is None else min_seq_length)
        self._max_seq_length = NumbersDict(sys.maxsize if max_seq_length is None else max_seq_length)

    def __iter__(self):
        for data_dict in self._dataset:
            lens = NumbersDict({k: v.shape[0] for k, v in data_dict.items() if isinstance(v, numpy.ndarray) and v.shape and v.dtype.kind not in "UO"})
            if self._min_seq_length.any_compare(lens, lambda a, b: a > b):
                continue
            if lens.any_compare(self._max_seq_length, lambda a, b: a > b):
                continue
            yield data_dict

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


class ShufflingDataPipe(torch.utils.data.IterableDataset):
    """
    Shuffle items through a buffer of ``buffer_size``. ``monotonic_data_keys`` (e.g. complete_frac, seq_idx) are
    re-assigned in sorted order so that they stay monotonic in the output stream.
    """

    def __init__(self, dataset: torch.utils.data.IterableDataset, *, buffer_size: int,
                 monotonic_data_keys: Sequence[str] = (), seed: Optional[int] = None):
        super().__init__()
        self._dataset = dataset
        self._buffer_size = buffer_size
        self._monotonic_data_keys = tuple(monotonic_data_keys)
        self._rng = numpy.random.RandomState()
        self._seed = seed % (2 ** 32) if seed is not None else None
        self._buffer: List[Any] = []
        self._next_buffer: List[Any] = []

    def set_seed(self, seed: int) -> "ShufflingDataPipe":
        """seed"""
        self._seed = seed % (2 ** 32)
        return self

    def __iter__(self):
        if self._seed is not None:
            self._rng.seed(self._seed)
        mono: Dict[str, List[Any]] = {k: [] for k in self._monotonic_data_keys}

        def _take(item):
            # items are batches (lists of dicts) or dicts
            vals = {}
            for k in self._monotonic_data_keys:
                if isinstance(item, dict) and k in item:
                    vals[k] = item[k]
            return vals

        def _emit(item, queue_vals):
            if isinstance(item, dict):
                for k, q in queue_vals.items():
                    if q and k in item:
                        item = dict(item)
                        item[k] = q.pop(0)
            return item

        buf: List[Any] = []
        for item in self._dataset:
            for k, v in _take(item).items():
                mono[k].append(v)
            if len(buf) < self._buffer_size:
                buf.append(item)
                continue
            idx = int(self._rng.randint(0, len(buf)))
            out = buf[idx]
            buf[idx] = item
            yield _emit(out, mono)
        self._rng.shuffle(buf)
        for out in buf:
            yield _emit(out, mono)

    def __getitem__(self, index):
        raise Exception("%s.__getitem__ not supported" % self.__class__.__name__)


def create_data_loader_from_batches(batches_dataset: torch.utils.data.Dataset, loader_opts: Optional[Dict[str, Any]] = None,
                                    *, packing: Optional[Dict[str, Any]] = None) -> torch.utils.data.DataLoader:
    """
    DataLoader over a dataset that already yields batches (lists of per-sequence dicts); ``collate_batch`` merges them.
    With ``num_workers > 0`` the workers are spawned (non-daemonic, so that datasets may spawn their own workers) and get
    the global config installed first.
    """
    import functools

    loader_opts = dict(loader_opts or {})
    if loader_opts.get("num_workers"):
        loader_opts.setdefault("persistent_workers", True)
        loader_opts.setdefault("worker_init_fn", _DataLoaderWorkerInitFunc())
        if "multiprocessing_context" not in loader_opts:
            from ...utils.multi_proc_non_daemonic_spawn import NonDaemonicSpawnContext
            from ...config import SubProcCopyGlobalConfigPreInitFunc

            loader_opts["multiprocessing_context"] = NonDaemonicSpawnContext(process_pre_init_func=SubProcCopyGlobalConfigPreInitFunc())
    collate = functools.partial(collate_batch, packing=packing) if packing is not None else collate_batch
    return torch.utils.data.DataLoader(batches_dataset, collate_fn=collate, batch_size=None, **loader_opts)


class _DataLoaderWorkerInitFunc:
    def __call__(self, worker_id: int):
        from ...utils import better_exchook

        better_exchook.install()
        try:
            import faulthandler

            faulthandler.enable()
        except Exception:
            pass
