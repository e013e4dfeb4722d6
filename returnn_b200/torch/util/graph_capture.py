"""
Whole-train-step CUDA-graph replay for user-defined RF models (config option ``torch_cuda_graph``).

A train step of a small or launch-bound model spends most of its time in the Python that issues its kernels. Here the step
(forward, losses, zeroing of the gradients, backward, optionally the optimizer update) is captured ONCE into a CUDA graph over
static, bound-shaped buffers and replayed for every batch:

* every ``extern_data`` key gets a device buffer ``[batch_size_bound, dim_capacity[key], ...]``; a batch is copied into
  its top-left corner (one ``copy_`` per key from the pinned host tensor), unused sequences have length 0;
* the sequence lengths live in static **device** int32 buffers and become the ``dyn_size_ext`` of the dynamic dims, so
  masks are computed on the device inside the graph (a model that reads a length on the host, e.g. ``int(lens.max())``,
  cannot be captured; the capture then fails with the CUDA error of the offending synchronisation);
* the losses are written to static scalars; ONE device-to-host copy per step reads them;
* the first ``warmup_steps`` steps run eagerly on a side stream (lazy initialisation: optimizer state, cuBLAS handles).

Options (``torch_cuda_graph`` dict): ``batch_size_bound`` (max. sequences per batch), ``dim_capacity`` (``{key: max
length}``), ``warmup_steps`` (default 2), ``capture_optimizer`` (default False: the optimizer runs eagerly on the static
gradients after the replay; True needs a capturable optimizer, e.g. the arena AdamW whose step counter is a device tensor).

With ``torch_distributed`` the captured part is forward + backward; the gradient reduction runs between the replay and the
eager optimizer step, which needs ``reduce_type="grad_explicit"`` (one flat reduction after backward) or ``"param"``:
the bucket hooks of ``"grad"`` cannot fire from a replayed graph, and ``capture_optimizer`` would put the update before the
reduction. Both combinations are rejected when the engine is set up.

The flagship models do not need this: their step is issued by the native encoder executor (one C call per
forward / backward range), which removes the Python between the kernels without the static-shape restriction.

Parity: returnn/torch/util/graph_capture.py (GraphCapturedTrainStep :410, run_train_step :1495, graph_pools_reserved :91).
The reference additionally offers an Inductor-compiled step; there is no tracing compiler here by design.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Tuple
import numpy
import torch

from ...tensor import Tensor, TensorDict, Dim, batch_dim
from ...utils.basic import NumbersDict, CollectionReadCheckCovered
from ...frontend._utils import dtype_name, torch_dtype
from ... import frontend as rf

_graphs: List["torch.cuda.CUDAGraph"] = []


def graph_pools_reserved() -> int:
    """
    :return: bytes held by the private memory pools of the captured graphs (they are invisible to
        ``torch.cuda.memory_allocated``'s "active" view after the capture; the engine's memory report adds them)
    """
    total = 0
    for g in _graphs:
        try:
            stats = torch.cuda.memory_stats()
            total = int(stats.get("reserved_bytes.all.current", 0)) - int(stats.get("active_bytes.all.current", 0))
            break
        except Exception:
            return 0
    return max(total, 0)


class GraphCapturedTrainStep:
    """eager warm-up steps, the one-time capture, per-step replay"""

    def __init__(self, *, engine, opts: Dict[str, Any]):
        """
        :param engine: the torch engine (gives the model, ``_run_step``, the updater, the extern_data template, the device)
        :param opts: see the module docstring
        """
        self.engine = engine
        device = str(engine._device)
        assert device.startswith("cuda"), "torch_cuda_graph requires a cuda device, got %r" % device
        opts = CollectionReadCheckCovered(dict(opts))
        self.batch_size_bound = int(opts["batch_size_bound"])
        self.dim_capacity: Dict[str, int] = dict(opts["dim_capacity"])
        self.warmup_steps = int(opts.get("warmup_steps", 2))
        self.capture_optimizer = bool(opts.get("capture_optimizer", False))
        opts.assert_all_read()
        dist = getattr(engine, "_torch_distributed_ctx", None)
        if dist is not None and dist.size() > 1:
            if dist.reduce_type == "grad":
                raise ValueError('torch_cuda_graph with torch_distributed needs reduce_type "grad_explicit" or "param": the bucket '
                                 'hooks of "grad" do not fire from a replayed graph')
            if self.capture_optimizer and dist.reduce_type != "param":
                raise ValueError("torch_cuda_graph: capture_optimizer=True would run the update before the gradient reduction")
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._len_bufs: Dict[str, torch.Tensor] = {}
        self._extern_data: Optional[TensorDict] = None
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._n_eager = 0
        self._loss_names: List[str] = []
        self._score_keys: set = set()
        self._loss_buf: Optional[torch.Tensor] = None  # [2 * n_losses]: summed losses, then inverse norm factors
        self._host_buf: Optional[torch.Tensor] = None
        self._stream = torch.cuda.Stream(device=device)
        self._params = [p for p in engine._pt_model.parameters() if p.requires_grad]

    # -- static buffers ----------------------------------------------------------------------------------------------
    def _build_extern_data(self) -> TensorDict:
        """template copies over the static buffers; dynamic dims sized by the static device length buffers"""
        eng = self.engine
        float_dtype = eng._default_float_dtype
        if isinstance(float_dtype, torch.dtype):
            float_dtype = dtype_name(float_dtype)
        res = TensorDict()
        bound = self.batch_size_bound
        batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(bound, dtype=torch.int32))
        for k, templ in eng.extern_data.data.items():
            if templ.dtype == "string":
                continue
            data = templ.copy_template()
            shape = []
            dyn_seen = False
            for dim in data.dims:
                if dim.is_batch_dim():
                    shape.append(bound)
                elif dim.is_static():
                    shape.append(dim.dimension)
                else:
                    assert not dyn_seen, "torch_cuda_graph: %r has more than one dynamic dim" % k
                    assert k in self.dim_capacity, "torch_cuda_graph: dim_capacity[%r] missing" % k
                    cap = int(self.dim_capacity[k])
                    shape.append(cap)
                    lens = torch.zeros(bound, dtype=torch.int32, device=self.device)
                    self._len_bufs[k] = lens
                    dim.dyn_size_ext = Tensor("%s:seq_len" % k, dims=[batch_dim], dtype="int32", raw_tensor=lens)
                    dim.capacity = cap
                    dyn_seen = True
            dtype = data.dtype
            if float_dtype and dtype.startswith("float"):
                dtype = float_dtype
                data.dtype = dtype
            buf = torch.zeros(shape, dtype=torch_dtype(dtype), device=self.device)
            self._bufs[k] = buf
            data._raw_tensor = buf
            res.data[k] = data
        return res

    def _copy_in(self, extern_data_raw: Dict[str, Any]):
        for k, buf in self._bufs.items():
            raw = extern_data_raw[k]
            if isinstance(raw, numpy.ndarray):
                raw = torch.from_numpy(raw)
            n = raw.shape[0]
            assert n <= self.batch_size_bound, "torch_cuda_graph: batch of %i seqs exceeds batch_size_bound %i" % (n, self.batch_size_bound)
            lens_buf = self._len_bufs.get(k)
            if lens_buf is not None:
                t = raw.shape[1]
                assert t <= buf.shape[1], "torch_cuda_graph: %r length %i exceeds dim_capacity %i" % (k, t, buf.shape[1])
                buf[:n, :t].copy_(raw, non_blocking=True)
                lens = extern_data_raw["%s:seq_len" % k]
                lens_buf.zero_()
                lens_buf[:n].copy_(lens.to(torch.int32), non_blocking=True)
                # stale frames beyond the new lengths are masked by the lengths; rows of unused sequences as well
            else:
                buf[:n].copy_(raw, non_blocking=True)

    # -- the step ----------------------------------------------------------------------------------------------------
    def _fwd_bwd(self):
        """forward + losses + backward on the static buffers; fills the static loss scalars"""
        eng = self.engine
        for p in self._params:
            if p.grad is not None:
                p.grad.zero_()
        # masks and derived sizes cached on the dims by an earlier step would be baked into the capture: recompute them from the
        # static length buffers inside this step (re-assigning the lengths invalidates the caches, also of derived dims)
        for data in self._extern_data.data.values():
            for dim in data.dims:
                if dim.is_dynamic() and not dim.is_batch_dim() and dim.dyn_size_ext is not None:
                    dim.dyn_size_ext = dim.dyn_size_ext
        eng._run_step(self._extern_data, train_flag=True, train_func=True)
        ctx = rf.get_run_ctx()
        names = list(ctx.losses.keys())
        if not self._loss_names:
            self._loss_names = names
            self._score_keys = set(k for k, v in ctx.losses.items() if not v.as_error)
            self._loss_buf = torch.zeros(2 * len(names), dtype=torch.float32, device=self.device)
            self._host_buf = torch.zeros(2 * len(names), dtype=torch.float32).pin_memory()
        assert names == self._loss_names, "torch_cuda_graph: the set of losses changed between steps"
        for i, n in enumerate(names):
            self._loss_buf[i].copy_(ctx.losses[n].get_summed_loss().raw_tensor.detach().float().reshape(()))
            f = ctx.losses[n].get_inv_norm_factor()
            if isinstance(f, Tensor):
                self._loss_buf[len(names) + i].copy_(f.raw_tensor.detach().float().reshape(()).to(self.device))
            else:
                self._loss_buf[len(names) + i].fill_(float(f))
        total = ctx.total_loss()
        if isinstance(total, Tensor) and total.raw_tensor.requires_grad:
            total.raw_tensor.backward()
        if self.capture_optimizer:
            eng._updater.step()

    def run_train_step(self, extern_data_raw: Dict[str, Any]) -> Tuple[NumbersDict, NumbersDict]:
        """
        :param extern_data_raw: the collated batch (host tensors)
        :return: summed losses, inverse norm factors (host numbers), as the eager step of the engine collects them
        """
        res = self.run_train_step_ex(extern_data_raw)
        n = len(res["names"])
        losses = NumbersDict({name: res["vals"][i] for i, name in enumerate(res["names"])})
        inv = NumbersDict({name: res["vals"][n + i] for i, name in enumerate(res["names"])})
        if self.engine._updater._log_grad_norm and res["grad_norm"] is not None:
            losses["grad_norm:p2"] = float(res["grad_norm"])
            inv["grad_norm:p2"] = 1.0
        return losses, inv

    def run_train_step_ex(self, extern_data_raw: Dict[str, Any], *, dist=None, epoch_step_idx: int = 0, read: bool = True) -> Dict[str, Any]:
        """
        One step: copy in, replay (or warm-up / capture), gradient reduction of the distributed context, optimizer, loss read.

        :param extern_data_raw: the collated batch (host tensors)
        :param dist: the engine's distributed context or None
        :param epoch_step_idx: step within the epoch (for the parameter-averaging schedule)
        :param read: False: the losses stay on the device (``vals`` is None then) and the host does not wait for the step
        :return: ``names`` (loss names), ``vals`` (host floats: the summed losses, then the inverse norm factors),
            ``score_keys`` (names that are scores, not errors), ``grad_norm`` (device scalar or None)
        """
        eng = self.engine
        if self._extern_data is None:
            self._extern_data = self._build_extern_data()
        self._copy_in(extern_data_raw)
        if self._graph is not None:
            self._graph.replay()
        elif self._n_eager < self.warmup_steps:
            self._n_eager += 1
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                self._fwd_bwd()
            torch.cuda.current_stream().wait_stream(self._stream)
        else:
            graph = torch.cuda.CUDAGraph()
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                # gradients must exist (and stay) as static tensors before the capture
                for p in self._params:
                    if p.grad is None:
                        p.grad = torch.zeros_like(p)
            torch.cuda.current_stream().wait_stream(self._stream)
            first_error: List[BaseException] = []
            try:
                with torch.cuda.graph(graph, stream=self._stream):
                    try:
                        self._fwd_bwd()
                    except BaseException as exc:  # the end of the capture raises its own error on top: keep the cause
                        first_error.append(exc)
            except Exception as exc:
                cause = first_error[0] if first_error else exc
                raise RuntimeError("torch_cuda_graph: the train step cannot be captured (an operation in it synchronises or copies from "
                                   "pageable host memory): %s: %s" % (type(cause).__name__, cause)) from cause
            if first_error:
                raise first_error[0]
            self._graph = graph
            _graphs.append(graph)
            graph.replay()
        if not self.capture_optimizer:
            if dist is not None:
                norm_sq = dist.maybe_reduce_grads(eng._pt_model)
                if norm_sq is not None:
                    eng._updater.set_precomputed_grad_norm_sq(norm_sq)
                dist.before_param_update(epoch_step_idx=epoch_step_idx)
            grad_norm = eng._updater.step()
        else:
            grad_norm = None
        if dist is not None:
            dist.step_after_param_update(module=eng._pt_model, epoch_step_idx=epoch_step_idx)
        if not read:
            return dict(names=list(self._loss_names), vals=None, score_keys=set(self._score_keys), grad_norm=grad_norm)
        self._host_buf.copy_(self._loss_buf, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return dict(names=list(self._loss_names), vals=self._host_buf.tolist(), score_keys=set(self._score_keys), grad_norm=grad_norm)
