"""
Legacy batch containers used by ``Dataset.generate_batches`` (in-dataset batching for tools and analysis).

Parity: returnn/engine/batch.py:1-381 (BatchSeqCopyPart, Batch, BatchSetGenerator).
"""

from __future__ import annotations
from typing import Sequence, Iterator, List, Optional
from ..utils.basic import NumbersDict


class BatchSeqCopyPart:
    """a slice of one sequence placed at (batch_slice, batch_frame_offset) of a batch"""

    def __init__(self, seq_idx: int, seq_start_frame, seq_end_frame, batch_slice: int, batch_frame_offset):
        self.seq_idx = seq_idx
        self.seq_start_frame = NumbersDict(seq_start_frame)
        self.seq_end_frame = NumbersDict(seq_end_frame)
        self.batch_slice = batch_slice
        self.batch_frame_offset = NumbersDict(batch_frame_offset)
        assert self.seq_start_frame.has_values() and self.seq_end_frame.has_values()

    @property
    def frame_length(self) -> NumbersDict:
        """frames per key"""
        return self.seq_end_frame - self.seq_start_frame

    def __repr__(self):
        return "<BatchSeqCopyPart seq %i frames %r..%r slice %i>" % (self.seq_idx, self.seq_start_frame, self.seq_end_frame, self.batch_slice)


class Batch:
    """a set of sequence parts; every part is its own slice (row)"""

    def __init__(self):
        self.max_num_frames_per_slice = NumbersDict(0)
        self.num_slices = 0
        self.seqs: List[BatchSeqCopyPart] = []

    def __repr__(self):
        return "<Batch start_seq:%r, len(seqs):%i>" % (self.start_seq, len(self.seqs))

    def try_sequence_as_slice(self, length) -> List:
        """:return: [new max frames per slice, new number of slices] if the sequence were added"""
        return [NumbersDict.max([self.max_num_frames_per_slice, length]), self.num_slices + 1]

    def add_sequence_as_slice(self, seq_idx: int, seq_start_frame, length):
        """add a part as a new slice"""
        length = NumbersDict(length)
        self.max_num_frames_per_slice, self.num_slices = self.try_sequence_as_slice(length)
        self.seqs.append(BatchSeqCopyPart(seq_idx=seq_idx, seq_start_frame=seq_start_frame, seq_end_frame=seq_start_frame + length,
                                          batch_slice=self.num_slices - 1, batch_frame_offset=0))

    def add_frames(self, seq_idx: int, seq_start_frame, length, frame_dim_corresponds: bool = True):
        """append to the single slice 0 (frame-wise training)"""
        length = NumbersDict(length)
        self.max_num_frames_per_slice += length
        self.num_slices = max(self.num_slices, 1)
        offset = self.max_num_frames_per_slice - length
        self.seqs.append(BatchSeqCopyPart(seq_idx=seq_idx, seq_start_frame=seq_start_frame, seq_end_frame=seq_start_frame + length,
                                          batch_slice=0, batch_frame_offset=offset))

    def init_with_one_full_sequence(self, seq_idx: int, dataset):
        """batch of exactly one full sequence"""
        assert not self.seqs
        start, end = dataset.get_start_end_frames_full_seq(seq_idx)
        self.add_frames(seq_idx=seq_idx, seq_start_frame=start, length=end - start)

    def get_all_slices_num_frames(self) -> NumbersDict:
        """padded frames"""
        return self.max_num_frames_per_slice * self.num_slices

    def get_total_num_frames(self) -> NumbersDict:
        """real frames"""
        total = NumbersDict(0)
        for s in self.seqs:
            total = total + s.frame_length
        return total

    @property
    def start_seq(self) -> Optional[int]:
        """first seq idx"""
        return min(s.seq_idx for s in self.seqs) if self.seqs else None

    @property
    def end_seq(self) -> Optional[int]:
        """last seq idx + 1"""
        return max(s.seq_idx for s in self.seqs) + 1 if self.seqs else None

    def get_num_seqs(self) -> int:
        """distinct sequences"""
        return 0 if not self.seqs else self.end_seq - self.start_seq


class BatchSetGenerator:
    """iterates over batches lazily with look-ahead; ``advance`` / ``peek_next_n`` / ``has_more``"""

    def __init__(self, dataset, generator: Iterator[Batch], shuffle_batches: bool = False, cache_whole_epoch: bool = True):
        self.dataset = dataset
        self.generator = generator
        self.shuffle_batches = shuffle_batches
        self.cache_whole_epoch = cache_whole_epoch
        self.cache: List[Batch] = []
        self.buffer: List[Batch] = []
        self.last_batch: Optional[Batch] = None
        self.reached_end = False
        self.current_batch_idx = 0
        self.reset()

    def reset(self):
        """restart (only possible when the whole epoch is cached)"""
        self.buffer = self.cache[:]
        self.current_batch_idx = 0
        self.reached_end = False
        self.last_batch = None
        if self.shuffle_batches and self.buffer:
            import random

            random.shuffle(self.buffer)

    def _read_next(self) -> bool:
        if self.reached_end:
            return False
        try:
            batch = next(self.generator)
        except StopIteration:
            self.reached_end = True
            return False
        self.last_batch = batch
        self.buffer.append(batch)
        if self.cache_whole_epoch:
            self.cache.append(batch)
        return True

    def _read_next_up_to_n(self, n: int):
        while len(self.buffer) < n:
            if not self._read_next():
                break

    def peek_next_n(self, n: int) -> List[Batch]:
        """next n batches without advancing"""
        self._read_next_up_to_n(n)
        return self.buffer[:n]

    def advance(self, n: int):
        """drop the first n"""
        self._read_next_up_to_n(n)
        self.buffer = self.buffer[n:]
        self.current_batch_idx += n

    def completed_frac(self) -> float:
        """progress estimate"""
        if self.cache_whole_epoch and self.reached_end and self.cache:
            return min(self.current_batch_idx / len(self.cache), 1.0)
        if self.last_batch is not None and self.last_batch.seqs:
            return self.dataset.get_complete_frac(self.last_batch.end_seq - 1) or 0.0
        return 0.0

    def has_more(self) -> bool:
        """any batch left"""
        if self.buffer:
            return True
        return self._read_next()

    def get_current_batch_idx(self) -> int:
        """index of the next batch"""
        return self.current_batch_idx


def batch_to_raw_dict(batch: Batch, *, dataset, extern_data=None, data_keys: Sequence[str], enforce_min_len1: bool = False, exclude_data_key=None):
    """
    The data of one :class:`Batch` out of the dataset as padded numpy arrays (chunks are sliced out of their sequences, frame-wise batches
    are laid out one after the other in slice 0). Backend independent: only the copy to a device differs between engines.

    :param extern_data: templates (``TensorDict``) that give the dtypes; the dataset's own dtypes if None
    :param exclude_data_key: function ``key -> bool``: keys to leave out
    :return: one ``[slices, max frames, ...]`` array per key, ``"<key>_seq_lens"`` per key with a time axis, ``"seq_idx"``, ``"seq_tag"``, ``"batch_dim"``
    Parity: returnn/engine/batch.py:290.
    """
    import numpy

    keys = [k for k in data_keys if not (exclude_data_key and exclude_data_key(k))]
    dataset.load_seqs(batch.start_seq, batch.end_seq)

    def dtype_of(k):
        if extern_data is not None and k in extern_data.data:
            return extern_data.data[k].dtype
        return dataset.get_data_dtype(k)

    n = batch.num_slices
    out, lens = {}, {}
    for k in keys:
        if dtype_of(k) == "string":
            out[k] = [""] * n
            continue
        t = int(batch.max_num_frames_per_slice[k])
        if enforce_min_len1:
            t = max(t, 1)
        shape = [n, t] + list(dataset.get_data_shape(k))
        out[k] = numpy.zeros(shape, dtype=dtype_of(k))
        lens[k] = numpy.zeros([n], dtype="int32")
    seq_idx, seq_tag = [-1] * n, [""] * n
    for part in batch.seqs:
        q = part.batch_slice
        seq_idx[q], seq_tag[q] = part.seq_idx, dataset.get_tag(part.seq_idx)
        for k in keys:
            data = dataset.get_data(part.seq_idx, k)
            if isinstance(out[k], list):
                out[k][q] = data if isinstance(data, str) else str(data)
                continue
            s0, s1 = int(part.seq_start_frame[k]), int(part.seq_end_frame[k])
            o = int(part.batch_frame_offset[k])
            ln = s1 - s0
            if ln > 0:
                chunk = data[s0:s1]
                out[k][q, o: o + chunk.shape[0]] = chunk  # a chunk that reaches past the sequence end leaves zeros
            lens[k][q] = max(int(lens[k][q]), o + ln)
    for k, v in lens.items():
        out["%s_seq_lens" % k] = v
    out["seq_idx"] = numpy.array(seq_idx, dtype="int32")
    out["seq_tag"] = numpy.array(seq_tag)
    out["batch_dim"] = numpy.array(n, dtype="int32")
    return out
