"""
Flat parameter arena: all parameters of a model live in one contiguous buffer per dtype (each ``nn.Parameter`` becomes a
view), and so do their gradients. Everything that touches "all weights" is then one pass over one pointer:
gradient all-reduce per bucket (a bucket is a contiguous slice), global grad norm, fused AdamW, parameter averaging.

Bucket order is reverse registration order (roughly the order in which autograd produces gradients), identical on
all ranks because it only depends on the module definition.
"""

from __future__ import annotations
from typing import Dict, Iterable, List, Optional, Sequence, Tuple
import torch

import weakref

_ALIGN = 128  # elements; keeps every tensor 512-byte aligned in fp32 (vector loads, TMA-able slices)
_arenas: "List[weakref.ref]" = []


def find_arena(t: torch.Tensor) -> "Optional[ParamArena]":
    """the live arena whose parameter buffer contains tensor ``t`` (None if there is none)"""
    addr = t.data_ptr()
    for ref in list(_arenas):
        a = ref()
        if a is None:
            _arenas.remove(ref)
            continue
        lo = a.flat_param.data_ptr()
        if a.flat_param.device == t.device and lo <= addr < lo + a.flat_param.numel() * a.flat_param.element_size():
            return a
    return None


class ArenaSlot:
    """where one parameter lives"""

    __slots__ = ("name", "param", "offset", "numel", "shape", "bucket")

    def __init__(self, name: str, param: torch.nn.Parameter, offset: int, numel: int):
        self.name = name
        self.param = param
        self.offset = offset
        self.numel = numel
        self.shape = tuple(param.shape)
        self.bucket = -1


class ParamArena:
    """
    Owns ``flat_param`` and ``flat_grad`` (same dtype and size) and re-points ``param.data`` / ``param.grad`` into them.
    """

    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], *, bucket_bytes: int = 32 << 20,
                 grad_dtype: Optional[torch.dtype] = None):
        params = [(n, p) for n, p in named_params if p.requires_grad]
        assert params, "ParamArena: no trainable parameters"
        self.device = params[0][1].device
        self.dtype = params[0][1].dtype
        for n, p in params:
            assert p.device == self.device and p.dtype == self.dtype, "ParamArena: mixed device/dtype at %r" % n
        self.slots: List[ArenaSlot] = []
        seen = set()
        offset = 0
        for n, p in params:
            if id(p) in seen:
                continue
            seen.add(id(p))
            numel = p.numel()
            self.slots.append(ArenaSlot(n, p, offset, numel))
            offset += (numel + _ALIGN - 1) // _ALIGN * _ALIGN
        self.total = offset
        self.flat_param = torch.zeros(self.total, dtype=self.dtype, device=self.device)
        self.grad_dtype = grad_dtype or self.dtype
        self.flat_grad = torch.zeros(self.total, dtype=self.grad_dtype, device=self.device)
        with torch.no_grad():
            for s in self.slots:
                view = self.flat_param[s.offset: s.offset + s.numel].view(s.shape)
                view.copy_(s.param.data)
                s.param.data = view
                if self.grad_dtype == self.dtype:
                    s.param.grad = self.flat_grad[s.offset: s.offset + s.numel].view(s.shape)
        # buckets: contiguous ranges, in reverse slot order
        elem = self.flat_grad.element_size()
        self.buckets: List[Tuple[int, int]] = []  # (start, end) element offsets, ordered by expected readiness
        end = self.total
        cur_end = end
        cur_bytes = 0
        n_in_bucket = 0
        for s in reversed(self.slots):
            cur_bytes += s.numel * elem
            n_in_bucket += 1
            if cur_bytes >= bucket_bytes:
                self.buckets.append((s.offset, cur_end))
                cur_end = s.offset
                cur_bytes = 0
                n_in_bucket = 0
        if cur_end > 0 and (n_in_bucket > 0 or not self.buckets):
            self.buckets.append((0, cur_end))
        for b, (lo, hi) in enumerate(self.buckets):
            for s in self.slots:
                if lo <= s.offset < hi:
                    s.bucket = b
        self.bucket_num_params = [sum(1 for s in self.slots if s.bucket == b) for b in range(len(self.buckets))]
        self._shadow: Optional[torch.Tensor] = None
        self._shadow_version = -1
        _arenas.append(weakref.ref(self))

    def shadow_bf16(self) -> torch.Tensor:
        """bf16 copy of ``flat_param`` (same element offsets): what the tensor-core GEMMs read. Allocated on first use."""
        if self._shadow is None:
            self._shadow = torch.empty(self.total, dtype=torch.bfloat16, device=self.device)
            self._shadow_version = -1
        return self._shadow

    def sync_shadow(self):
        """
        Bring the bf16 copy up to date if the fp32 weights changed through torch since the last sync (checkpoint load,
        initialisation, parameter averaging). An optimizer kernel that writes both copies itself calls
        :func:`mark_shadow_synced` instead, so the steady state costs nothing here.
        """
        sh = self.shadow_bf16()
        v = self.flat_param._version
        if v != self._shadow_version:
            with torch.no_grad():
                sh.copy_(self.flat_param)
            self._shadow_version = self.flat_param._version

    def mark_shadow_synced(self):
        """the caller has just written fp32 weights and bf16 copy together"""
        self._shadow_version = self.flat_param._version

    def has_shadow(self) -> bool:
        """whether a bf16 copy is being maintained"""
        return self._shadow is not None

    def replace_grad_buffer(self, new_flat: torch.Tensor):
        """
        Move the gradient arena into ``new_flat`` (same dtype, at least ``total`` elements; e.g. symmetric memory that
        peer GPUs can address) and re-point every ``param.grad`` into it.
        """
        assert new_flat.dtype == self.grad_dtype and new_flat.numel() >= self.total and new_flat.device == self.device
        new_flat = new_flat[: self.total]
        with torch.no_grad():
            new_flat.copy_(self.flat_grad)
        self.flat_grad = new_flat
        if self.grad_dtype == self.dtype:
            for s in self.slots:
                s.param.grad = self.flat_grad[s.offset: s.offset + s.numel].view(s.shape)

    def replace_param_buffer(self, new_flat: torch.Tensor):
        """move the parameter arena into ``new_flat`` (e.g. symmetric memory) and re-point every ``param.data`` into it"""
        assert new_flat.dtype == self.dtype and new_flat.numel() >= self.total and new_flat.device == self.device
        new_flat = new_flat[: self.total]
        with torch.no_grad():
            new_flat.copy_(self.flat_param)
            self.flat_param = new_flat
            for s in self.slots:
                s.param.data = self.flat_param[s.offset: s.offset + s.numel].view(s.shape)
        self._shadow_version = -1

    def invalidate_shadow(self):
        """the fp32 weights were changed by a kernel that bypasses torch's version counter"""
        self._shadow_version = -1

    def zero_grad(self):
        """one memset for all gradients"""
        self.flat_grad.zero_()

    def grad_view(self, slot: "ArenaSlot") -> torch.Tensor:
        """the view of the gradient arena that belongs to one parameter"""
        return self.flat_grad[slot.offset: slot.offset + slot.numel].view(slot.shape)

    def relink_grads(self):
        """make sure every ``param.grad`` is the arena view (autograd may have replaced it when it was None)"""
        if self.grad_dtype != self.dtype:
            return
        base = self.flat_grad.data_ptr()
        views = getattr(self, "_grad_views", None)
        if views is None or self._grad_views_base != base:
            # one view object per parameter, kept: the common case below is then an identity check per parameter
            views = [self.flat_grad[s.offset: s.offset + s.numel].view(s.shape) for s in self.slots]
            self._grad_views, self._grad_views_base = views, base
        for s, view in zip(self.slots, views):
            g = s.param.grad
            if g is view:
                continue
            if g is None:
                s.param.grad = view
            elif g.data_ptr() != view.data_ptr():
                view.copy_(g)
                s.param.grad = view
            else:
                s.param.grad = view

    def bucket_grad(self, b: int) -> torch.Tensor:
        """gradient slice of bucket b"""
        lo, hi = self.buckets[b]
        return self.flat_grad[lo:hi]

    def bucket_param(self, b: int) -> torch.Tensor:
        """parameter slice of bucket b"""
        lo, hi = self.buckets[b]
        return self.flat_param[lo:hi]

    def nbytes(self) -> int:
        """bytes of one flat buffer"""
        return self.total * self.flat_param.element_size()
