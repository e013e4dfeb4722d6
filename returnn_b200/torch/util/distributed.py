"""
Differentiable all-reduce: forward all-reduces the value, backward all-reduces the gradient (for statistics that every
rank contributes to, e.g. synchronised BatchNorm).

Parity: returnn/torch/util/distributed.py:13-58.
"""

from __future__ import annotations
import torch
import torch.distributed as dist

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "avg": dist.ReduceOp.SUM}


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        out = x.clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM)
        return g


def all_reduce_differentiable(x: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """all-reduce over the default group; identity when not distributed"""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return x
    if op in ("sum", "avg"):
        out = _AllReduceSum.apply(x)
        if op == "avg":
            out = out / dist.get_world_size()
        return out
    out = x.detach().clone()
    dist.all_reduce(out, op=_OPS[op])
    return out


all_reduce_sum = all_reduce_differentiable
