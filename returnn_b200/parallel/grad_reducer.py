"""
Bucketed gradient all-reduce overlapped with backward (``reduce_type="grad"``).

A post-accumulate-grad hook per parameter counts down its bucket; when the bucket is complete, the reduction of that
contiguous gradient slice is launched on a side stream while autograd continues with earlier layers. On B200 with
peer access the reduction is the fused NVLink kernel of :mod:`returnn_b200.parallel.fused_allreduce` (peer loads,
scale by 1/N, running sum of squares for the global grad norm); otherwise ``torch.distributed.all_reduce`` (NCCL/Gloo).
``finish()`` joins the side stream and returns the squared global gradient norm when the fused path produced it.
"""

from __future__ import annotations
from typing import List, Optional
import torch
import torch.distributed as dist
from .arena import ParamArena


_active: "Optional[BucketedGradReducer]" = None


def get_active() -> "Optional[BucketedGradReducer]":
    """the reducer of this process (there is at most one), for code that writes gradients without autograd hooks"""
    return _active


def notify_grads_written(tensors):
    """
    Tell the active reducer that the gradients of these parameters are complete. ``tensors`` are parameters, or views of the
    gradient arena; used by ops that accumulate into the arena directly, where no post-accumulate-grad hook fires.
    """
    r = _active
    if r is None:
        return
    r.mark_ready(tensors)


class BucketedGradReducer:
    """drives per-bucket reductions from autograd hooks"""

    def __init__(self, arena: ParamArena, *, process_group=None, fused=None, average: bool = True):
        self.arena = arena
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.average = average
        self.fused = fused  # object with reduce_bucket(b, lo, hi, stream) / finish(), or None
        self._pending = list(arena.bucket_num_params)
        self._works: List = []
        self._enabled = True
        self._stream: Optional[torch.cuda.Stream] = torch.cuda.Stream(device=arena.device) if arena.device.type == "cuda" else None
        self._handles = []
        self._launched = [False] * len(arena.buckets)
        for s in arena.slots:
            self._handles.append(s.param.register_post_accumulate_grad_hook(self._make_hook(s)))
        self._counted = set()
        global _active
        _active = self

    def mark_ready(self, tensors):
        """gradients written outside autograd: parameters (views of ``flat_param``) or gradient views (of ``flat_grad``)"""
        if not self._enabled or self.world == 1:
            return
        a = self.arena
        p0, g0 = a.flat_param.data_ptr(), a.flat_grad.data_ptr()
        pe, ge = a.flat_param.element_size(), a.flat_grad.element_size()
        if not hasattr(self, "_slot_by_offset"):
            self._slot_by_offset = {s.offset: s for s in a.slots}
        for t in tensors:
            if t is None:
                continue
            addr = t.data_ptr()
            if p0 <= addr < p0 + a.total * pe:
                off = (addr - p0) // pe
            elif g0 <= addr < g0 + a.total * ge:
                off = (addr - g0) // ge
            else:
                continue
            s = self._slot_by_offset.get(off)
            if s is None or off in self._counted:
                continue
            self._counted.add(off)
            self._pending[s.bucket] -= 1
            if self._pending[s.bucket] == 0 and not self._launched[s.bucket]:
                self._launch(s.bucket)

    def _make_hook(self, slot):
        b = slot.bucket
        arena = self.arena

        def hook(param):
            if not self._enabled or self.world == 1:
                return
            # The bucket reduction reads the arena slice. If this gradient was accumulated into a tensor of its own (the
            # gradient was None when backward started, e.g. after a zero_grad(set_to_none=True)), move it into the arena and
            # re-point param.grad BEFORE the bucket counts down: otherwise the reduction would run on stale arena contents.
            if arena.grad_dtype == arena.dtype:
                g = param.grad
                if g is not None:
                    view = arena.grad_view(slot)
                    if g.data_ptr() != view.data_ptr():
                        view.copy_(g)
                        param.grad = view
            self._pending[b] -= 1
            if self._pending[b] == 0:
                self._launch(b)

        return hook

    def set_enabled(self, enabled: bool):
        """False during gradient accumulation micro-steps (no_sync)"""
        self._enabled = enabled

    def prepare_backward(self):
        """reset the per-bucket counters"""
        self._pending = list(self.arena.bucket_num_params)
        self._works = []
        self._launched = [False] * len(self.arena.buckets)
        self._counted = set()

    def _launch(self, b: int):
        self._launched[b] = True
        lo, hi = self.arena.buckets[b]
        g = self.arena.flat_grad[lo:hi]
        if self.fused is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                self.fused.reduce_bucket(b, lo, hi)
            return
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                if self.average:
                    g.div_(self.world)
                self._works.append(dist.all_reduce(g, group=self.pg, async_op=True))
        else:
            if self.average:
                g.div_(self.world)
            self._works.append(dist.all_reduce(g, group=self.pg, async_op=True))

    def finish(self) -> Optional[torch.Tensor]:
        """
        Wait for all bucket reductions; buckets whose hooks never fired (unused parameters) are reduced now.
        :return: squared global grad norm (device scalar) if the fused path computed it, else None
        """
        if self.world == 1 or not self._enabled:
            return None
        for b, done in enumerate(self._launched):
            if not done:
                self._launch(b)
        for w in self._works:
            w.wait()
        self._works = []
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)
        if self.fused is not None:
            return self.fused.finish()
        return None

    def remove(self):
        """unregister hooks"""
        global _active
        for h in self._handles:
            h.remove()
        self._handles = []
        if _active is self:
            _active = None
