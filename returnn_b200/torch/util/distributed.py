"""
Differentiable all-reduce: forward all-reduces the value, backward all-reduces the gradient (for statistics that every
rank contributes to, e.g. synchronised BatchNorm).

Parity: returnn/torch/util/distributed.py:13-58.
"""

from __future__ import annotations
import torch
import torch.distributed as dist

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "avg": dist.ReduceOp.SUM}


def _sum_over_ranks(x: torch.Tensor) -> torch.Tensor:
    """small fp32 CUDA vectors (batch-norm statistics) go through the one-kernel NVLink exchange, everything else through NCCL / gloo"""
    if x.is_cuda:
        from ...parallel import fused_allreduce as _far

        red = _far.get_small_reducer()
        if red is not None and red.supports(x):
            return red.all_reduce_sum(x.contiguous())
    out = x.clone()
    dist.all_reduce(out, op=dist.ReduceOp.SUM)
    return out


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _sum_over_ranks(x)

    @staticmethod
    def backward(ctx, g):
        return _sum_over_ranks(g)


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


def all_reduce_sum(x: torch.Tensor) -> torch.Tensor:
    """sum over the ranks, differentiable (the gradient is summed over the ranks as well); identity without a process group"""
    return all_reduce_differentiable(x, op="sum")
