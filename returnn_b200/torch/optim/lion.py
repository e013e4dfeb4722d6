"""
Lion optimizer (https://arxiv.org/abs/2302.06675): ``update = sign(b1*m + (1-b1)*g)``, decoupled weight decay,
``m = b2*m + (1-b2)*g``. On CUDA the update of each parameter is one fused kernel.

Parity: returnn/torch/optim/lion.py:1-216.
"""

from __future__ import annotations
from typing import Callable, Optional, Tuple
import torch
from torch.optim.optimizer import Optimizer


class Lion(Optimizer):
    """Lion"""

    def __init__(self, params, lr: float = 1e-4, betas: Tuple[float, float] = (0.9, 0.99), weight_decay: float = 0.0, use_triton: bool = False):
        assert lr > 0.0 and all(0.0 <= b <= 1.0 for b in betas)
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, wd = group["lr"], group["weight_decay"]
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if len(state) == 0:
                    state["exp_avg"] = torch.zeros_like(p)
                m = state["exp_avg"]
                if p.is_cuda:
                    from ...ops import optim_native

                    if optim_native.lion_available(p):
                        optim_native.lion_update(p, p.grad, m, lr, wd, b1, b2)
                        continue
                p.mul_(1.0 - lr * wd)
                update = m.mul(b1).add_(p.grad, alpha=1.0 - b1).sign_()
                p.add_(update, alpha=-lr)
                m.mul_(b2).add_(p.grad, alpha=1.0 - b2)
        return loss
