"""
:class:`DistributeFilesDataset`: a very large dataset given as a list of files (or a nested structure of files).
Every sub-epoch a slice of the files is turned into a sub dataset by the user's ``get_sub_epoch_dataset(files_subepoch)``;
under distributed training every rank gets its own slice of the files of the sub-epoch (sharding by file, balanced by
file size); the files of the *next* sub-epoch are copied to the local cache in the background
(reference: returnn/datasets/distrib_files.py:37).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union
import os
import threading
import numpy
from .basic import Dataset, DatasetSeq, init_dataset
from .cached2 import CachedDataset2
from ..log import log

FileTree = Union[str, Sequence["FileTree"], Dict[Any, "FileTree"]]


def _flatten(tree: FileTree) -> List[str]:
    if isinstance(tree, str):
        return [tree]
    if isinstance(tree, dict):
        return [f for v in tree.values() for f in _flatten(v)]
    return [f for v in tree for f in _flatten(v)]


def _get_key_file(tree: FileTree) -> str:
    return _flatten(tree)[0]


class DistributeFilesDataset(CachedDataset2):
    """files → sub-epoch datasets, sharded over ranks"""

    def __init__(self, files: Union[Sequence[FileTree], Callable[[], Sequence[FileTree]]], get_sub_epoch_dataset: Callable[[List[FileTree]], Dict[str, Any]],
                 preload_next_n_sub_epochs: int = 1, buffer_size: int = 1, distrib_shard_files: Optional[bool] = None, file_cache_opts: Optional[Dict[str, Any]] = None,
                 _meta_info_cache: Optional[Dict[str, Any]] = None, _distrib_info: Optional[Dict[str, int]] = None, **kwargs):
        super().__init__(**kwargs)
        self._files_arg = files
        self._files: Optional[List[FileTree]] = None
        self.get_sub_epoch_dataset = get_sub_epoch_dataset
        self.preload_next_n_sub_epochs = preload_next_n_sub_epochs
        self.distrib_shard_files = distrib_shard_files
        self._file_cache_opts = file_cache_opts
        self._file_cache = None
        self._sub: Optional[Dataset] = None
        self._file_sizes: Optional[Dict[str, int]] = None
        self._distrib_info = _distrib_info
        self._preload_threads: Dict[int, threading.Thread] = {}
        self._meta = _meta_info_cache
        self.num_outputs = None
        if self._meta:
            self._apply_meta(self._meta)

    def _apply_meta(self, meta: Dict[str, Any]):
        self.num_inputs, self.num_outputs, self.labels = meta["num_inputs"], meta["num_outputs"], meta["labels"]
        self._keys, self._targets, self._dtypes = meta["keys"], meta["targets"], meta["dtypes"]

    def initialize(self):
        """meta information (data keys, dims) comes from a first sub dataset unless it was cached"""
        self._need_meta()
        super().initialize()

    def _lazy_files(self) -> List[FileTree]:
        if self._files is None:
            files = self._files_arg() if callable(self._files_arg) else self._files_arg
            self._files = list(files)
            assert self._files, "%s: no files" % self
        return self._files

    def _rank_and_size(self) -> Tuple[int, int]:
        if self._distrib_info:
            return self._distrib_info["rank"], self._distrib_info["size"]
        if self._num_shards > 1:
            return self._shard_index, self._num_shards
        try:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                return dist.get_rank(), dist.get_world_size()
        except ImportError:
            pass
        return 0, 1

    def _size_of(self, tree: FileTree) -> int:
        if self._file_sizes is None:
            self._file_sizes = {}
        key = _get_key_file(tree)
        if key not in self._file_sizes:
            try:
                self._file_sizes[key] = max(os.path.getsize(key), 1)
            except OSError:
                self._file_sizes[key] = 1
        return self._file_sizes[key]

    def files_for_sub_epoch(self, epoch: int) -> List[FileTree]:
        """the files of sub-epoch ``epoch`` for this rank"""
        files = self._lazy_files()
        pe = max(self.partition_epoch, 1)
        full_epoch = (epoch - 1) // pe + 1
        part = (epoch - 1) % pe
        order = self.get_seq_order_for_epoch(epoch=full_epoch, num_seqs=len(files), get_seq_len=lambda i: self._size_of(files[i]))
        # partition_epoch was applied by get_seq_order_for_epoch when given the sub-epoch; here we want the same order for
        # all parts of one full epoch, so cut it ourselves
        order = list(order)
        if len(order) != len(files):  # the base class already partitioned: recompute the cut from the full order
            order = list(range(len(files)))
        rank, size = self._rank_and_size()
        shard = self.distrib_shard_files if self.distrib_shard_files is not None else size > 1
        if shard and size > 1:
            # one cut into partition_epoch * size chunks: sub-epoch `part` of rank r is chunk part * size + r
            assert len(order) >= pe * size, "%s: %i files for %i sub-epochs x %i ranks" % (self, len(order), pe, size)
            mine = self._split_by_size(order, pe * size, files)[part * size + rank]
        else:
            mine = self._split_by_size(order, pe, files)[part]
        return [files[i] for i in mine]

    def _split_by_size(self, idxs: Sequence[int], n: int, files: List[FileTree]) -> List[List[int]]:
        """n contiguous chunks of about equal total file size, none empty"""
        idxs = list(idxs)
        assert len(idxs) >= n
        sizes = numpy.array([self._size_of(files[i]) for i in idxs], dtype="float64")
        total = sizes.sum()
        bounds, acc, k = [0], 0.0, 1
        for j, s in enumerate(sizes):
            acc += s
            remaining_items = len(idxs) - (j + 1)
            remaining_chunks = n - k
            if k < n and (acc >= total * k / n or remaining_items == remaining_chunks):
                bounds.append(j + 1)
                k += 1
        while len(bounds) < n:
            bounds.append(bounds[-1] + 1)
        bounds.append(len(idxs))
        return [idxs[bounds[i]: bounds[i + 1]] for i in range(n)]

    def _cache_files(self, tree: FileTree) -> FileTree:
        if self._file_cache_opts is None:
            return tree
        if self._file_cache is None:
            from ..utils.file_cache import FileCache

            self._file_cache = FileCache(**self._file_cache_opts)
        if isinstance(tree, str):
            return self._file_cache.get_file(tree)
        if isinstance(tree, dict):
            return {k: self._cache_files(v) for k, v in tree.items()}
        return type(tree)(self._cache_files(v) for v in tree)

    def _preload(self, epoch: int):
        if self._file_cache_opts is None or epoch in self._preload_threads:
            return

        def run():
            try:
                for f in self.files_for_sub_epoch(epoch):
                    self._cache_files(f)
            except Exception as exc:
                print("%s: preloading sub-epoch %i failed: %s" % (self, epoch, exc), file=log.v2)

        t = threading.Thread(target=run, name="%s preload %i" % (self.name, epoch), daemon=True)
        t.start()
        self._preload_threads[epoch] = t

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        assert seq_list is None and seq_order is None, "%s: explicit orders are not supported" % self
        if epoch is None:
            self._num_seqs = 0
            return True
        t = self._preload_threads.pop(epoch, None)
        if t is not None:
            t.join()
        files = [self._cache_files(f) for f in self.files_for_sub_epoch(epoch)]
        opts = self.get_sub_epoch_dataset(files)
        self._sub = init_dataset(opts, parent_dataset=self)
        self._sub.init_seq_order(epoch=epoch)
        if self.num_outputs is None:
            ds = self._sub
            self._apply_meta({"num_inputs": ds.num_inputs, "num_outputs": ds.num_outputs, "labels": ds.labels, "keys": ds.get_data_keys(),
                              "targets": ds.get_target_list(), "dtypes": {k: ds.get_data_dtype(k) for k in ds.get_data_keys()}})
        for e in range(epoch + 1, epoch + 1 + self.preload_next_n_sub_epochs):
            self._preload(e)
        self._num_seqs = None
        return True

    def supports_sharding(self) -> bool:
        return True

    @property
    def num_seqs(self) -> int:
        return self._sub.num_seqs if self._sub is not None else 0

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        ds = self._sub
        if ds is None or not ds.is_less_than_num_seqs(seq_idx):
            return None
        ds.load_seqs(seq_idx, seq_idx + 1)
        return DatasetSeq(seq_idx=seq_idx, seq_tag=ds.get_tag(seq_idx), features={k: ds.get_data(seq_idx, k) for k in ds.get_data_keys()})

    def _need_meta(self):
        if self.num_outputs is None:
            files = self.files_for_sub_epoch(1)
            ds = init_dataset(self.get_sub_epoch_dataset([self._cache_files(f) for f in files[:1]]), parent_dataset=self)
            self._apply_meta({"num_inputs": ds.num_inputs, "num_outputs": ds.num_outputs, "labels": ds.labels, "keys": ds.get_data_keys(),
                              "targets": ds.get_target_list(), "dtypes": {k: ds.get_data_dtype(k) for k in ds.get_data_keys()}})

    def get_data_keys(self):
        self._need_meta()
        return list(self._keys)

    def get_target_list(self):
        self._need_meta()
        return list(self._targets)

    def get_data_dtype(self, key):
        self._need_meta()
        return self._dtypes[key]

    def get_data_dim(self, key):
        self._need_meta()
        return self.num_outputs[key][0]

    def is_data_sparse(self, key):
        self._need_meta()
        return self.num_outputs[key][1] == 1

    def get_data_shape(self, key):
        return [] if self.is_data_sparse(key) else [self.num_outputs[key][0]]
