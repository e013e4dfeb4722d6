"""
:class:`PostprocessingDataset`: apply user functions to the sequences of a wrapped dataset, per sequence
(``map_seq(tensor_dict, *, epoch, seq_idx, rng, **_) -> tensor_dict``) and/or on the stream
(``map_seq_stream(iterator, *, epoch, rng, **_) -> iterator``), e.g. speed perturbation, filtering, concatenation, or
re-ordering with :class:`LaplaceOrdering` (reference: returnn/datasets/postprocessing.py:36, 911).
"""

from __future__ import annotations
from ..utils.basic import OptionalNotImplementedError
from typing import Any, Callable, Dict, Iterator, List, Optional
import numpy
from .basic import Dataset, DatasetSeq, init_dataset
from .cached2 import CachedDataset2
from ..tensor import Tensor, Dim, TensorDict, batch_dim
from ..utils.basic import get_fwd_compat_kwargs


class PostprocessingDataset(CachedDataset2):
    """wrapped dataset + mapping functions"""

    def __init__(self, dataset: Dict[str, Any], map_seq: Optional[Callable] = None, map_seq_stream: Optional[Callable] = None,
                 map_outputs: Optional[Dict[str, Any]] = None, map_seq_stream_preserves_num_seqs: Optional[bool] = None,
                 buf_size: int = 1, num_workers: int = 0, **kwargs):
        super().__init__(**kwargs)
        if self.seq_ordering != "default":
            raise ValueError("%s: specify seq_ordering in the wrapped dataset" % self)
        if map_seq is None and map_seq_stream is None:
            raise ValueError("%s: need map_seq or map_seq_stream" % self)
        self._dataset_def = dataset
        self._map_seq = map_seq
        self._map_seq_stream = map_seq_stream
        self._map_outputs = map_outputs
        self._preserves_num_seqs = map_seq_stream_preserves_num_seqs if map_seq_stream_preserves_num_seqs is not None else (map_seq_stream is None)
        self._rng = numpy.random.RandomState(0)
        self._dataset = init_dataset(dataset, parent_dataset=self)
        self._iter: Optional[Iterator[TensorDict]] = None
        self.labels = dict(self._dataset.labels)
        if map_outputs is not None:
            self._out_template = TensorDict()
            self._out_template.update(map_outputs, auto_convert=True)
        else:
            self._out_template = self._template_of(self._dataset)
        self.num_outputs = {k: (t.sparse_dim.dimension if t.sparse_dim else (t.shape[-1] if t.shape else 1) or 1, t.ndim)
                            for k, t in self._out_template.data.items()}
        self.num_inputs = self.num_outputs.get("data", (0, 0))[0]

    @staticmethod
    def _template_of(ds: Dataset) -> TensorDict:
        td = TensorDict()
        for key in ds.get_data_keys():
            dims = [Dim(None, name="%s_time" % key)]
            sparse = None
            if ds.is_data_sparse(key):
                sparse = Dim(ds.get_data_dim(key), name="%s_classes" % key)
                dims += [Dim(d, name="%s_dim%i" % (key, i)) for i, d in enumerate(ds.get_data_shape(key)[1:])]
            else:
                shape = ds.get_data_shape(key)
                dims += [Dim(d, name="%s_dim%i" % (key, i)) for i, d in enumerate(shape)]
            td.data[key] = Tensor(key, dims=dims, dtype=ds.get_data_dtype(key), sparse_dim=sparse)
        return td

    def get_current_seq_order(self):
        """the order of the wrapped dataset (a stream function that changes the number of sequences has no such order)"""
        if not self._preserves_num_seqs:
            raise OptionalNotImplementedError("%s: map_seq_stream may change the sequences" % self)
        return self._dataset.get_current_seq_order()

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if epoch is None and seq_list is None and seq_order is None:
            self._num_seqs = 0
            return True
        self._dataset.init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        self._rng = numpy.random.RandomState(self._get_random_seed_for_epoch(epoch=epoch))
        self._iter = self._build_iter()
        self._num_seqs = None
        return True

    def _source_iter(self) -> Iterator[TensorDict]:
        ds = self._dataset
        template = self._template_of(ds)
        i = 0
        while ds.is_less_than_num_seqs(i):
            ds.load_seqs(i, i + 1)
            td = TensorDict()
            for key, t in template.data.items():
                t2 = t.copy_template()
                t2.raw_tensor = ds.get_data(i, key)
                td.data[key] = t2
            tag = Tensor("seq_tag", dims=[], dtype="string")
            tag.raw_tensor = numpy.array(ds.get_tag(i))
            td.data["seq_tag"] = tag
            if self._map_seq is not None:
                td = self._map_seq(td, epoch=self.epoch, seq_idx=i, rng=self._rng, **get_fwd_compat_kwargs())
                assert isinstance(td, TensorDict), "%s: map_seq must return a TensorDict, got %r" % (self, type(td))
                if "seq_tag" not in td.data:
                    td.data["seq_tag"] = tag
            yield td
            i += 1

    def _build_iter(self) -> Iterator[TensorDict]:
        it = self._source_iter()
        if self._map_seq_stream is not None:
            it = self._map_seq_stream(it, epoch=self.epoch, rng=self._rng, **get_fwd_compat_kwargs())
        return iter(it)

    @property
    def num_seqs(self) -> int:
        if self._preserves_num_seqs:
            return self._dataset.num_seqs
        if self._num_seqs is not None:
            return self._num_seqs
        raise NotImplementedError("%s: number of sequences unknown until the stream is exhausted" % self)

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        if self._preserves_num_seqs:
            return self._dataset.get_total_num_seqs(fast=fast)
        raise NotImplementedError

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if self._iter is None:
            return None
        try:
            td = next(self._iter)
        except StopIteration:
            self._num_seqs = seq_idx
            return None
        tag = td.data.get("seq_tag")
        tag_s = str(tag.raw_tensor) if tag is not None and tag.raw_tensor is not None else "seq-%i" % seq_idx
        feats = {k: numpy.asarray(v.raw_tensor) for k, v in td.data.items() if k != "seq_tag" and k in self._out_template.data}
        return DatasetSeq(seq_idx=seq_idx, seq_tag=tag_s, features=feats)

    def get_data_keys(self):
        return list(self._out_template.data.keys())

    def get_target_list(self):
        return [k for k in self.get_data_keys() if k != "data"]

    def get_data_dtype(self, key):
        return self._out_template.data[key].dtype

    def get_data_dim(self, key):
        return self.num_outputs[key][0]

    def is_data_sparse(self, key):
        return self._out_template.data[key].sparse_dim is not None

    def get_data_shape(self, key):
        t = self._out_template.data[key]
        return [d.dimension for d in t.dims[1:]]


class LaplaceOrdering:
    """
    ``map_seq_stream`` that sorts buffers of ``num_seqs_per_bin`` sequences by length, alternating direction per bin
    (the streaming counterpart of ``seq_ordering="laplace"``; reference: returnn/datasets/postprocessing.py:911).
    """

    def __init__(self, num_seqs_per_bin: int, length_key: str = "data"):
        assert num_seqs_per_bin > 0
        self.num_seqs_per_bin = num_seqs_per_bin
        self.length_key = length_key

    def __call__(self, iterator: Iterator[TensorDict], **kwargs) -> Iterator[TensorDict]:
        buf: List[TensorDict] = []
        ascending = True
        for td in iterator:
            buf.append(td)
            if len(buf) >= self.num_seqs_per_bin:
                buf.sort(key=lambda t: t.data[self.length_key].raw_tensor.shape[0], reverse=not ascending)
                yield from buf
                buf = []
                ascending = not ascending
        buf.sort(key=lambda t: t.data[self.length_key].raw_tensor.shape[0], reverse=not ascending)
        yield from buf
