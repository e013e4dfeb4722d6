"""
AdamW over the flat parameter arena: one kernel reads gradient, weights and both moments once and writes weights and
moments (plus, optionally, a bf16 copy of the weights for the next forward). The global-norm clip coefficient is
applied inside the same kernel, so clipping costs no extra pass.

``FusedArenaAdamW`` behaves like a ``torch.optim.Optimizer`` (param_groups with ``lr``, ``state_dict`` /
``load_state_dict``, ``zero_grad``), so the Updater and the checkpoint code treat it like any other optimizer.
On CPU (tests) the same math runs in torch.
"""

from __future__ import annotations
from typing import Any, Dict, Iterable, List, Optional, Set, Tuple
import ctypes
import math
import torch
from ...parallel.arena import ParamArena


def fused_available(device: torch.device) -> bool:
    """the native kernel can be used on this device"""
    if device.type != "cuda":
        return False
    from ...ops import _lib

    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_adamw_arena")


class FusedArenaAdamW(torch.optim.Optimizer):
    """Adam / AdamW on a ParamArena"""

    is_fused_arena = True

    def __init__(self, network: torch.nn.Module, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 decoupled: bool = True, weight_decay_param_names: Optional[Set[str]] = None, arena: Optional[ParamArena] = None):
        named = [(n, p) for n, p in network.named_parameters() if p.requires_grad]
        if arena is None:
            arena = ParamArena(named)
        self.arena = arena
        self._names = [s.name for s in arena.slots]
        super().__init__([s.param for s in arena.slots], dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))
        self.decoupled = decoupled
        dev, n = arena.device, arena.total
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        # per-element weight-decay mask as a per-slot table: decay flag per 128-element block
        wd_names = weight_decay_param_names
        flags = torch.zeros((n + 127) // 128, dtype=torch.uint8)
        for s in arena.slots:
            if wd_names is None or s.name in wd_names:
                flags[s.offset // 128: (s.offset + s.numel + 127) // 128] = 1
        self.wd_flags = flags.to(dev)
        self.step_count = 0
        self._step_t = torch.zeros(1, dtype=torch.int64, device=dev)
        self._clip = 0.0
        self._norm: Optional[torch.Tensor] = None
        self._scratch = torch.zeros(1024 + 8, dtype=torch.float32, device=dev)

    def param_names(self) -> List[str]:
        """names in slot order"""
        return list(self._names)

    def zero_grad(self, set_to_none: bool = False):
        """memset of the gradient arena (views stay linked)"""
        self.arena.zero_grad()

    def grad_norm(self) -> torch.Tensor:
        """global L2 norm of the gradient arena (device scalar)"""
        self.arena.relink_grads()
        g = self.arena.flat_grad
        if g.is_cuda:
            from ...ops import optim_native

            if optim_native.available():
                return torch.sqrt(optim_native.sum_squares(g, self._scratch))
        return torch.linalg.vector_norm(g.float(), 2.0)

    def set_clip(self, max_norm: float, norm: torch.Tensor):
        """clip coefficient min(1, max_norm / (norm + 1e-6)) applied in the next step()"""
        self._clip = float(max_norm)
        self._norm = norm

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.arena.relink_grads()
        group = self.param_groups[0]
        lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
        self.step_count += 1
        t = self.step_count
        bc1 = 1.0 - b1 ** t
        bc2 = 1.0 - b2 ** t
        p, g, m, v = self.arena.flat_param, self.arena.flat_grad, self.exp_avg, self.exp_avg_sq
        if p.is_cuda:
            from ...ops import optim_native

            avg = getattr(self, "param_averager", None)
            if avg is not None and avg.pending:
                # sync step of the parameter-averaging mode: update and average in one kernel over NVLink
                avg.average(dict(g=g, m=m, v=v, wd_flags=self.wd_flags, lr=lr, b1=b1, b2=b2, eps=eps, wd=wd, bc1=bc1, bc2=bc2,
                                 decoupled=self.decoupled, clip=self._clip if self._norm is not None else 0.0, norm=self._norm))
                self._norm = None
                return loss
            if optim_native.available():
                optim_native.adamw_arena(p, g, m, v, self.wd_flags, lr=lr, b1=b1, b2=b2, eps=eps, wd=wd, bc1=bc1, bc2=bc2,
                                         decoupled=self.decoupled, clip=self._clip if self._norm is not None else 0.0, norm=self._norm,
                                         p_bf16=self.arena.shadow_bf16() if self.arena.has_shadow() else None)
                if self.arena.has_shadow():
                    self.arena.mark_shadow_synced()
                self._norm = None
                return loss
        gg = g.float()
        if self._norm is not None and self._clip:
            gg = gg * torch.clamp(self._clip / (self._norm + 1e-6), max=1.0)
        self._norm = None
        mask = self.wd_flags.repeat_interleave(128)[: p.numel()].to(torch.bool)
        if wd and not self.decoupled:
            gg = gg + wd * p.float() * mask
        m.mul_(b1).add_(gg, alpha=1.0 - b1)
        v.mul_(b2).addcmul_(gg, gg, value=1.0 - b2)
        denom = (v / bc2).sqrt_().add_(eps)
        upd = (m / bc1) / denom
        if wd and self.decoupled:
            p.mul_(torch.where(mask, torch.full((), 1.0 - lr * wd, device=p.device), torch.ones((), device=p.device)).to(p.dtype))
        p.add_(upd.to(p.dtype), alpha=-lr)
        return loss

    def state_dict(self) -> Dict[str, Any]:
        """per-parameter ``exp_avg`` / ``exp_avg_sq`` / ``step`` like torch.optim.AdamW, so that files are interchangeable"""
        state = {}
        for i, s in enumerate(self.arena.slots):
            state[i] = {
                "step": torch.tensor(float(self.step_count)),
                "exp_avg": self.exp_avg[s.offset: s.offset + s.numel].view(s.shape).clone(),
                "exp_avg_sq": self.exp_avg_sq[s.offset: s.offset + s.numel].view(s.shape).clone(),
            }
        g = dict(self.param_groups[0])
        g["params"] = list(range(len(self.arena.slots)))
        return {"state": state, "param_groups": [g]}

    def load_state_dict(self, state_dict: Dict[str, Any]):
        """accepts its own format and that of torch.optim.Adam(W) with the same parameter order"""
        st = state_dict["state"]
        step = 0
        for i, s in enumerate(self.arena.slots):
            if i in st:
                self.exp_avg[s.offset: s.offset + s.numel].view(s.shape).copy_(st[i]["exp_avg"])
                self.exp_avg_sq[s.offset: s.offset + s.numel].view(s.shape).copy_(st[i]["exp_avg_sq"])
                step = max(step, int(float(st[i]["step"])))
        self.step_count = step
        if state_dict.get("param_groups"):
            g = state_dict["param_groups"][0]
            for k in ("lr", "betas", "eps", "weight_decay"):
                if k in g:
                    self.param_groups[0][k] = g[k]
