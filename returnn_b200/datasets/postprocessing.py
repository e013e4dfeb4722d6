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
        if buf_size < 1:
            raise ValueError("%s: buf_size must be > 0, got %r" % (self, buf_size))
        if num_workers < 0:
            raise ValueError("%s: num_workers must be >= 0, got %r" % (self, num_workers))
        if map_seq_stream_preserves_num_seqs is None and map_seq_stream is not None:
            map_seq_stream_preserves_num_seqs = getattr(map_seq_stream, "preserves_num_seqs", None)
        self._buf_size = buf_size
        self._num_workers = num_workers
        self._workers: Optional["_WorkerPool"] = None
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
        if self._num_workers > 0:
            if self._workers is None:
                template = {k: dict(name=k, dims=list(t.dims), dtype=t.dtype, sparse_dim=t.sparse_dim) for k, t in self._template_of(self._dataset).data.items()}
                self._workers = _WorkerPool(self._num_workers, self._buf_size, self._map_seq, self._map_seq_stream, template, name=str(self))
            self._iter = self._workers.start_epoch(self._raw_source_iter(), epoch=self.epoch, seed=self._get_random_seed_for_epoch(epoch=epoch))
        else:
            self._iter = self._build_iter()
        self._num_seqs = None
        return True

    def finish_epoch(self, *, free_resources: bool = False):
        super().finish_epoch(free_resources=free_resources)
        if self._workers is not None:
            self._workers.end_epoch()
            if free_resources:
                self._workers.close()
                self._workers = None

    def __del__(self):
        workers = getattr(self, "_workers", None)
        if workers is not None:
            workers.close()

    def _raw_source_iter(self) -> Iterator[Dict[str, numpy.ndarray]]:
        """the wrapped dataset's sequences as plain arrays (what travels to the worker processes)"""
        ds = self._dataset
        i = 0
        while ds.is_less_than_num_seqs(i):
            ds.load_seqs(i, i + 1)
            item = {key: ds.get_data(i, key) for key in ds.get_data_keys()}
            item["seq_tag"] = numpy.array(ds.get_tag(i))
            yield item
            i += 1

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
        tag = td.data.get("seq_tag") if not isinstance(td, dict) else None
        tag_s = str(tag.raw_tensor) if tag is not None and tag.raw_tensor is not None else "seq-%i" % seq_idx
        if isinstance(td, dict):  # from a worker process: plain arrays
            tag_s = str(td["seq_tag"]) if "seq_tag" in td else "seq-%i" % seq_idx
            return DatasetSeq(seq_idx=seq_idx, seq_tag=tag_s, features={k: numpy.asarray(v) for k, v in td.items() if k != "seq_tag" and k in self._out_template.data})
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


def _arrays_to_tensor_dict(item: Dict[str, numpy.ndarray], template: Dict[str, Any]) -> TensorDict:
    td = TensorDict()
    for key, raw in item.items():
        if key == "seq_tag":
            t = Tensor("seq_tag", dims=[], dtype="string")
        else:
            t = template[key].copy_template()
        t.raw_tensor = numpy.asarray(raw)
        td.data[key] = t
    return td


def _tensor_dict_to_arrays(td: TensorDict) -> Dict[str, numpy.ndarray]:
    return {k: numpy.asarray(v.raw_tensor) for k, v in td.data.items()}


def _worker_main(worker_idx: int, conn, feed_conn, setup: bytes, buf_size: int):
    """
    One worker process. It pulls its share of the input sequences from the parent's feeder (request / reply on ``feed_conn``),
    applies the mapping functions, and answers the parent's ``next`` requests on ``conn``, computing up to ``buf_size`` results
    ahead while no request is pending.
    """
    from collections import deque
    import pickle
    from ..utils import better_exchook

    better_exchook.install()
    map_seq, map_seq_stream, template_kwargs = pickle.loads(setup)
    template = {k: Tensor(**kw) for k, kw in template_kwargs.items()}
    out_iter: Optional[Iterator[TensorDict]] = None
    buffer: deque = deque()
    exhausted = True
    try:
        while True:
            if out_iter is not None and not exhausted and len(buffer) < buf_size and not conn.poll(0):
                try:
                    buffer.append(("seq", _tensor_dict_to_arrays(next(out_iter))))
                except StopIteration:
                    exhausted = True
                    buffer.append(("end", None))
                continue
            msg, arg = conn.recv()
            if msg == "exit":
                return
            if msg == "epoch":
                epoch, seed, generation = arg
                rng = numpy.random.RandomState((seed * 683859 + worker_idx * 4099) % (2 ** 31))
                buffer.clear()
                exhausted = False

                def source(epoch=epoch, rng=rng, generation=generation):
                    while True:
                        feed_conn.send(("get", generation))
                        kind, item = feed_conn.recv()
                        if kind == "end":
                            return
                        seq_idx = item.pop("__seq_idx__")
                        td = _arrays_to_tensor_dict(item, template)
                        if map_seq is not None:
                            tag = td.data.get("seq_tag")
                            td = map_seq(td, epoch=epoch, seq_idx=seq_idx, rng=rng, **get_fwd_compat_kwargs())
                            assert isinstance(td, TensorDict), "map_seq must return a TensorDict, got %r" % (type(td),)
                            if "seq_tag" not in td.data and tag is not None:
                                td.data["seq_tag"] = tag
                        yield td

                it = source()
                if map_seq_stream is not None:
                    it = map_seq_stream(it, epoch=epoch, rng=rng, **get_fwd_compat_kwargs())
                out_iter = iter(it)
            elif msg == "next":
                while not buffer:
                    try:
                        buffer.append(("seq", _tensor_dict_to_arrays(next(out_iter))))
                    except StopIteration:
                        exhausted = True
                        buffer.append(("end", None))
                conn.send(buffer.popleft() if buffer[0][0] != "end" else buffer[0])
            else:
                raise ValueError("unknown message %r" % (msg,))
    except (EOFError, BrokenPipeError, KeyboardInterrupt):
        return  # the parent went away
    except BaseException as exc:
        import traceback

        try:
            conn.send(("exc", "%s: %s\n%s" % (type(exc).__name__, exc, traceback.format_exc())))
        except Exception:
            pass


class _WorkerPool:
    """
    ``num_workers`` processes that apply the mapping functions. Input sequence ``i`` goes to worker ``i % num_workers``, and
    results are taken from the workers in turn, so with a per-sequence function the order of the wrapped dataset is kept. A
    feeder thread in this process reads the wrapped dataset and serves the workers' requests; what it reads for a worker that has
    not asked yet waits in that worker's queue. The functions travel with the by-value pickler, so they may come from a config file.
    (reference: returnn/datasets/postprocessing.py:446 feeder, :817 worker loop)
    """

    def __init__(self, num_workers: int, buf_size: int, map_seq, map_seq_stream, template: Dict[str, Dict[str, Any]], *,
                 name: str = "PostprocessingDataset"):
        from ..utils.multi_proc_non_daemonic_spawn import NonDaemonicSpawnContext
        from ..utils import task_system

        self.num_workers = num_workers
        self.name = name
        ctx = NonDaemonicSpawnContext(process_pre_init_func=None)
        self._conns = []
        self._feed_conns = []
        self._procs = []
        self._feeder = None
        self._feeder_stop = False
        self._setup_args = (map_seq, map_seq_stream, template)
        self._generation = 0
        self._feeder_exc: Optional[BaseException] = None
        self._task_system = task_system
        self._ctx = ctx
        self._buf_size = buf_size
        self._started = False
        self._active: List[int] = []
        self._turn = 0

    def _start_procs(self):
        setup = self._task_system.dumps(self._setup_args)
        for i in range(self.num_workers):
            parent_conn, child_conn = self._ctx.Pipe()
            feed_parent, feed_child = self._ctx.Pipe()
            proc = self._ctx.Process(target=_worker_main, args=(i, child_conn, feed_child, setup, self._buf_size),
                                     name="%s worker %i" % (self.name, i), daemon=True)
            proc.start()
            child_conn.close()
            feed_child.close()
            self._conns.append(parent_conn)
            self._feed_conns.append(feed_parent)
            self._procs.append(proc)
        self._started = True

    def start_epoch(self, source: Iterator[Dict[str, numpy.ndarray]], *, epoch: int, seed: int) -> Iterator[Dict[str, numpy.ndarray]]:
        """new epoch over ``source``; returns the iterator over the results"""
        import threading

        self.end_epoch()
        source = iter(source)
        if not self._started:
            self._start_procs()
        self._generation += 1
        for conn in self._conns:
            conn.send(("epoch", (epoch, seed, self._generation)))
        self._feeder_stop = False
        self._feeder = threading.Thread(target=self._feed, args=(source, self._generation), name="%s feeder" % self.name, daemon=True)
        self._feeder.start()
        self._active = list(range(self.num_workers))
        self._turn = 0
        return self._results()

    def _feed(self, source: Iterator[Dict[str, numpy.ndarray]], generation: int):
        from multiprocessing.connection import wait
        from collections import deque

        queues = [deque() for _ in range(self.num_workers)]
        next_idx = 0
        source_done = False
        open_conns = {conn: i for i, conn in enumerate(self._feed_conns)}
        finished = set()
        try:
            while not self._feeder_stop and len(finished) < self.num_workers:
                ready = wait(list(open_conns.keys()), timeout=0.1)
                for conn in ready:
                    w = open_conns[conn]
                    try:
                        _, req_generation = conn.recv()
                    except (EOFError, OSError):
                        finished.add(w)
                        del open_conns[conn]
                        continue
                    if req_generation != generation:
                        conn.send(("end", None))  # a request of the epoch before: that stream is over
                        continue
                    while not queues[w] and not source_done:
                        item = next(source, None)
                        if item is None:
                            source_done = True
                            break
                        item = dict(item)
                        item["__seq_idx__"] = next_idx
                        queues[next_idx % self.num_workers].append(item)
                        next_idx += 1
                    if queues[w]:
                        conn.send(("seq", queues[w].popleft()))
                    else:
                        conn.send(("end", None))
                        finished.add(w)
        except Exception as exc:  # noqa
            self._feeder_exc = exc

    def _results(self) -> Iterator[Dict[str, numpy.ndarray]]:
        while self._active:
            self._turn %= len(self._active)
            w = self._active[self._turn]
            conn = self._conns[w]
            conn.send(("next", None))
            while not conn.poll(1.0):
                if not self._procs[w].is_alive():
                    raise RuntimeError("%s: worker %i died (exit code %r)" % (self.name, w, self._procs[w].exitcode))
                if self._feeder_exc is not None:
                    raise RuntimeError("%s: reading the wrapped dataset failed" % self.name) from self._feeder_exc
            kind, item = conn.recv()
            if kind == "exc":
                raise RuntimeError("%s: worker %i failed:\n%s" % (self.name, w, item))
            if kind == "end":
                self._active.pop(self._turn)
                continue
            self._turn += 1
            yield item

    def end_epoch(self):
        """stop the feeder of the running epoch"""
        if self._feeder is not None:
            self._feeder_stop = True
            self._feeder.join(timeout=5.0)
            self._feeder = None

    def close(self):
        """stop the processes"""
        self.end_epoch()
        for conn in self._feed_conns:  # a worker that waits for input sees the end of the pipe
            try:
                conn.close()
            except Exception:
                pass
        for conn in self._conns:
            try:
                conn.send(("exit", None))
            except Exception:
                pass
        for proc in self._procs:
            proc.join(timeout=2.0)
            if proc.is_alive():
                proc.terminate()
        for conn in self._conns + self._feed_conns:
            try:
                conn.close()
            except Exception:
                pass
        self._conns, self._feed_conns, self._procs = [], [], []
        self._started = False


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


class Sequential:
    """
    Composition of post-processing functions: ``Sequential(f, g)(x) == g(f(x))``. Works for ``map_seq`` functions (one sequence in, one
    out) and for ``map_seq_stream`` functions (iterator in, iterator out); the two kinds are not to be mixed in one instance.
    Keyword arguments (``epoch``, ``rng`` ...) are handed to every function. Parity: returnn/datasets/postprocessing.py:975.
    """

    def __init__(self, *postprocessing_funcs: Callable):
        self.funcs = postprocessing_funcs

    def __call__(self, arg, **kwargs):
        for func in self.funcs:
            arg = func(arg, **kwargs)
        return arg

    @property
    def preserves_num_seqs(self) -> bool:
        """whether every composed function says of itself that it maps sequences one to one"""
        return all(getattr(f, "preserves_num_seqs", False) for f in self.funcs)
