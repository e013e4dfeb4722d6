"""
Distributed (data-parallel) context for the torch engine. Config key ``torch_distributed`` (dict):

- ``backend``: process-group backend string; default ``"cpu:gloo,cuda:nccl"`` on GPU, ``"gloo"`` on CPU
- ``timeout_sec``: collective timeout (default 1800)
- ``reduce_type``: ``"grad"`` (bucketed gradient reduction overlapped with backward; default),
  ``"grad_explicit"`` (one flat reduction after backward), ``"param"`` (independent workers, parameters averaged
  every ``param_sync_step`` steps)
- ``param_sync_step``: for ``"param"``
- ``sync_on_cpu``: do the parameter averaging through host memory (Gloo)
- ``class`` / ``options``: wrap the module with a user class (e.g. ``torch.nn.parallel.DistributedDataParallel``)
  instead of the built-in reducer
- ``fused``: ``True`` / ``False`` / ``None`` (auto): use the fused NVLink kernels (peer loads over NVSwitch from inside
  the reduction kernel, fused with scaling and grad-norm partial sums; parameter averaging fused with AdamW) when every
  rank is a B200 on one node. ``False`` keeps the NCCL baseline.
- ``bucket_cap_mb``: bucket size for ``"grad"`` (default 32)
- ``fused_wait_ms``: time limit of the cross-rank waits inside the fused kernels (default 20000, or the environment variable
  ``RETURNN_B200_COLLECTIVE_WAIT_MS``). A kernel whose peer does not arrive in time gives up and reports through the status
  board; the engine raises ``KernelWaitTimeout`` one step later.

One process per GPU, started by ``torchrun`` (RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR/PORT from the environment).

Parity: returnn/torch/distributed.py:22-238 (DistributedContext, _sync_params_avg :211-238, get_ctx :185-208).
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Union
import datetime
import os
import socket
import torch
import torch.distributed as dist
from ..config import Config
from ..log import log
from ..utils.basic import CollectionReadCheckCovered

_ctx: Optional["DistributedContext"] = None


class DistributedContext:
    """process group + reduce-type logic"""

    def __init__(self, options: Dict[str, Any]):
        self._opts = CollectionReadCheckCovered(options)
        self._local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self._local_size = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
        backend = self._opts.get("backend", None)
        timeout = datetime.timedelta(seconds=self._opts.get("timeout_sec", 1800))
        if not dist.is_initialized():
            if backend is None:
                backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
            if "MASTER_ADDR" not in os.environ:
                os.environ["MASTER_ADDR"] = "127.0.0.1"
                os.environ.setdefault("MASTER_PORT", "29500")
                os.environ.setdefault("RANK", "0")
                os.environ.setdefault("WORLD_SIZE", "1")
            if torch.cuda.is_available():
                torch.cuda.set_device(self._local_rank % max(torch.cuda.device_count(), 1))
            dist.init_process_group(backend=backend, timeout=timeout)
        self._rank = dist.get_rank()
        self._size = dist.get_world_size()
        self._reduce_type = self._opts.get("reduce_type", "grad")
        self._param_sync_step: Optional[int] = self._opts.get("param_sync_step", None)
        if self._reduce_type == "param":
            assert isinstance(self._param_sync_step, int) and self._param_sync_step > 0, (
                "reduce_type param: param_sync_step must be a positive int")
        self._sync_on_cpu = self._opts.get("sync_on_cpu", False)
        self._custom_class = self._opts.get("class", None)
        self._custom_class_opts = self._opts.get("options", None)
        self._fused_opt = self._opts.get("fused", None)
        self._bucket_cap_mb = self._opts.get("bucket_cap_mb", 32)
        self._fused_wait_ms = self._opts.get("fused_wait_ms", None)
        peer_watch_opts = self._opts.get("peer_watch", None)
        self._opts.assert_all_read()
        from ..parallel import peer_watch as _peer_watch

        # host-side liveness of the peers (heartbeats in the process group's store), checked before every step
        self.peer_watch = _peer_watch.create_from_process_group(peer_watch_opts, rank=self._rank, world=self._size)
        self._reducer = None
        self._arena = None
        self._fused = None
        self._param_averager = None
        self._step_after_param_update_module = None
        print("Torch distributed initialized. Hostname %s, pid %i, rank %i / size %i, local rank %s / local size %s, reduce_type %s." % (
            socket.gethostname(), os.getpid(), self._rank, self._size, self._local_rank, self._local_size, self._reduce_type), file=log.v3)

    def check_peers(self, step: Optional[int] = None):
        """raises ``parallel.peer_watch.PeerFailure`` when a peer left or went silent; call before issuing a step"""
        if self.peer_watch is not None:
            self.peer_watch.check(step)

    def leave_job(self, reason: str = "left"):
        """
        this rank leaves on purpose: only between steps. Waits for the device (nothing of this rank may be in flight), then
        tells the peers through the store.
        """
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()
        if self.peer_watch is not None:
            self.peer_watch.leave(reason)

    def local_rank(self) -> int:
        """rank on this node"""
        return self._local_rank

    def local_size(self) -> int:
        """processes on this node"""
        return self._local_size

    def rank(self) -> int:
        """global rank"""
        return self._rank

    def size(self) -> int:
        """world size"""
        return self._size

    @property
    def reduce_type(self) -> str:
        """grad / grad_explicit / param"""
        return self._reduce_type

    def get_param_sync_step(self) -> Optional[int]:
        """N for parameter averaging"""
        return self._param_sync_step

    def want_fused(self, device: torch.device) -> bool:
        """whether to try the fused NVLink kernels"""
        if self._fused_opt is False or device.type != "cuda" or self._size == 1:
            return False
        if self._size != self._local_size:
            if self._fused_opt:
                raise ValueError("torch_distributed fused=True needs all ranks on one node")
            return False
        if self._sync_on_cpu:
            return False
        return True

    def maybe_make_distributed_module(self, module: torch.nn.Module) -> Optional[torch.nn.Module]:
        """
        For ``reduce_type="grad"`` with a custom ``class``: wrap the module (its forward runs the whole train step).
        With the built-in reducer nothing is wrapped: :func:`setup_grad_reduction` installs hooks instead.
        """
        if self._reduce_type != "grad" or self._custom_class is None:
            return None
        cls = self._custom_class
        if isinstance(cls, str):
            import importlib

            mod_name, _, cls_name = cls.rpartition(".")
            cls = getattr(importlib.import_module(mod_name), cls_name)
        kwargs = dict(self._custom_class_opts or {})
        if cls is torch.nn.parallel.DistributedDataParallel and module_device(module).type == "cuda":
            kwargs.setdefault("device_ids", [self._local_rank])
        return cls(module, **kwargs)

    def setup_grad_reduction(self, module: torch.nn.Module):
        """
        Built-in path for ``"grad"`` and ``"grad_explicit"``: flatten parameters into an arena, broadcast the initial
        weights from rank 0, and (for ``"grad"``) install the bucket hooks.
        """
        from ..parallel.arena import ParamArena
        from ..parallel.grad_reducer import BucketedGradReducer

        if self._size == 1:
            return
        for p in module.parameters():
            dist.broadcast(p.data, src=0)
        for b in module.buffers():
            if b.is_floating_point():
                dist.broadcast(b.data, src=0)
        if self._reduce_type == "param" and self._custom_class is None and self.want_fused(module_device(module)):
            named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
            if len({p.dtype for _, p in named}) == 1:
                from ..parallel import fused_allreduce

                self._arena = ParamArena(named, bucket_bytes=int(self._bucket_cap_mb) << 20)
                self._param_averager = fused_allreduce.try_create_param_averager(
                    self._arena, rank=self._rank, world=self._size, required=bool(self._fused_opt), wait_ms=self._fused_wait_ms)
            return
        if self._reduce_type not in ("grad", "grad_explicit") or self._custom_class is not None:
            return
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        dtypes = {p.dtype for _, p in named}
        if len(dtypes) != 1:
            return  # mixed dtypes: fall back to per-parameter reduction in maybe_reduce_grads
        self._arena = ParamArena(named, bucket_bytes=int(self._bucket_cap_mb) << 20)
        device = self._arena.device
        if self.want_fused(device):
            from ..parallel import fused_allreduce

            self._fused = fused_allreduce.try_create(self._arena, rank=self._rank, world=self._size, required=bool(self._fused_opt),
                                                     wait_ms=self._fused_wait_ms)
            from ..config import get_global_config

            cfg = get_global_config(raise_exception=False)
            if (self._fused is not None and cfg is not None and cfg.bool("rf_batch_norm_distributed", False)
                    and os.environ.get("RETURNN_B200_SMALL_ALLREDUCE", "0") == "1"):
                # cross-rank batch-norm statistics: a one-kernel exchange of the [C] sums instead of a library collective.
                # Opt-in: measured on 2 GPUs it takes 160 us per call (copy in, one-CTA kernel with two cross-GPU flag rounds,
                # copy out) against 108 us for NCCL on the same 4 KB vector.
                fused_allreduce.try_create_small_reducer(device=device, rank=self._rank, world=self._size)
        if self._reduce_type == "grad":
            self._reducer = BucketedGradReducer(self._arena, fused=self._fused)

    @property
    def arena(self):
        """the flat parameter arena, if the built-in reduction is active"""
        return self._arena

    @property
    def fused(self):
        """the fused NVLink reducer, if active"""
        return self._fused

    @property
    def grad_reduce_mode(self) -> str:
        """
        how gradients (or parameters, for ``reduce_type="param"``) cross the GPUs: ``"fused-multimem"`` (own kernel, reduction inside
        the NVSwitch), ``"fused-peer"`` (own kernel, peer loads and stores), ``"nccl"`` / ``"gloo"`` (library collective), ``"none"``
        """
        if self._size == 1:
            return "none"
        f = self._fused if self._fused is not None else self._param_averager
        if f is not None:
            return f.mode
        return "nccl" if (self._arena is not None and self._arena.device.type == "cuda") or torch.cuda.is_available() else "gloo"

    def prepare_backward(self, *, sync: bool = True):
        """before ``loss.backward()``; ``sync=False`` for gradient accumulation micro-steps"""
        if self._reducer is not None:
            self._reducer.set_enabled(sync)
            if sync:
                self._reducer.prepare_backward()

    def maybe_reduce_grads(self, module: torch.nn.Module) -> Optional[torch.Tensor]:
        """
        After backward: finish the bucket reductions (``"grad"``) or reduce everything now (``"grad_explicit"``).
        :return: squared global grad norm if the fused kernels produced it
        """
        if self._size == 1:
            return None
        if self._reduce_type == "grad":
            if self._reducer is not None:
                self._arena.relink_grads()
                return self._reducer.finish()
            if self._custom_class is None:
                self._reduce_per_param(module)
            return None
        if self._reduce_type == "grad_explicit":
            if self._arena is not None:
                self._arena.relink_grads()
                if self._fused is not None:
                    self._fused.reduce_bucket(0, 0, self._arena.total)
                    return self._fused.finish()
                g = self._arena.flat_grad
                dist.all_reduce(g)
                g.div_(self._size)
            else:
                self._reduce_per_param(module)
        return None

    def _reduce_per_param(self, module: torch.nn.Module):
        grads = [p.grad for p in module.parameters() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat)
        flat.div_(self._size)
        off = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[off: off + n].view_as(g))
            off += n

    def should_sync_now(self, *, epoch_step_idx: int) -> bool:
        """whether this step does a parameter sync"""
        if self._reduce_type != "param":
            return False
        return epoch_step_idx % self._param_sync_step == self._param_sync_step - 1

    @property
    def param_averager(self):
        """the fused parameter averager (``reduce_type="param"`` on one NVLink node), if active"""
        return self._param_averager

    def before_param_update(self, *, epoch_step_idx: int):
        """
        Called before the optimizer step. On sync steps of the fused parameter-averaging mode this marks the averager as pending,
        so that the arena optimizer runs its update inside the averaging kernel.
        """
        if self._param_averager is not None and self.should_sync_now(epoch_step_idx=epoch_step_idx):
            self._param_averager.pending = True

    def step_after_param_update(self, *, module: torch.nn.Module, epoch_step_idx: int):
        """parameter averaging when due"""
        if self._reduce_type == "param" and self.should_sync_now(epoch_step_idx=epoch_step_idx):
            if self._param_averager is not None:
                if self._param_averager.pending:  # the optimizer did not fuse it (other optimizer class): average only
                    self._param_averager.average(None)
                return
            _sync_params_avg(module=module, sync_on_cpu=self._sync_on_cpu, ctx=self)


def module_device(module: torch.nn.Module) -> torch.device:
    """device of the first parameter"""
    for p in module.parameters():
        return p.device
    return torch.device("cpu")


def get_ctx(config: Optional[Config] = None) -> Optional[DistributedContext]:
    """the process-wide context, created from config ``torch_distributed`` on first use; None if not configured"""
    global _ctx
    if _ctx is not None:
        return _ctx
    if not config:
        from ..config import get_global_config

        config = get_global_config(raise_exception=False)
        if not config:
            return None
    opts = config.typed_value("torch_distributed")
    if opts is None:
        return None
    assert isinstance(opts, dict)
    _ctx = DistributedContext(opts)
    return _ctx


def reset_ctx():
    """forget the context (tests)"""
    global _ctx
    _ctx = None


def _sync_params_avg(*, module: torch.nn.Module, sync_on_cpu: bool = False, ctx: Optional[DistributedContext] = None):
    """
    Average all parameters over the ranks: one collective over a flat buffer (not one per tensor).
    On B200 peers the fused kernel does it in place through peer loads.
    """
    params = [p for p in module.parameters()]
    if not params:
        return
    size = dist.get_world_size()
    with torch.no_grad():
        if ctx is not None and ctx.arena is not None and not sync_on_cpu and len(ctx.arena.slots) == len([p for p in params if p.requires_grad]):
            flat = ctx.arena.flat_param
            dist.all_reduce(flat)
            flat.div_(size)
            return
        flat = torch.cat([p.data.reshape(-1).float() for p in params])
        if sync_on_cpu:
            flat_cpu = flat.cpu()
            dist.all_reduce(flat_cpu)
            flat = flat_cpu.to(flat.device)
        else:
            dist.all_reduce(flat)
        flat.div_(size)
        off = 0
        for p in params:
            n = p.numel()
            p.data.copy_(flat[off: off + n].view_as(p))
            off += n
