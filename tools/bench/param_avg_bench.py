"""
Value check and timing of the fused AdamW + parameter-averaging kernel on the GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29521 \\
        tools/bench/param_avg_bench.py [--elems 50000000]

Every rank starts from the same weights, takes one AdamW step on its own (rank-dependent) gradients inside the fused kernel
and receives the average. The result is compared with the same computation done with torch ops + ``dist.all_reduce``;
both are timed (CUDA events, max over ranks). Rank 0 prints one JSON line.
"""

from __future__ import annotations
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import argparse
import json
import os
import sys
import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elems", type=int, default=50_000_000)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from returnn_b200.parallel.arena import ParamArena
    from returnn_b200.parallel import fused_allreduce
    from returnn_b200.torch.optim.fused_adamw import FusedArenaAdamW

    torch.manual_seed(0)
    net = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(args.elems // 2 + 7, device=dev) * 0.1),
                                  torch.nn.Parameter(torch.randn(args.elems // 2, device=dev) * 0.1)])
    module = torch.nn.Module()
    module.ps = net
    opt = FusedArenaAdamW(module, lr=1e-2, weight_decay=0.01)
    arena = opt.arena
    avg = fused_allreduce.FusedParamAverager(arena, rank=rank, world=world)
    opt.param_averager = avg
    start = arena.flat_param.clone()
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    grads = torch.randn(arena.total, device=dev, generator=g)

    def reference():
        # one AdamW step from zero moments, then the average over ranks
        b1, b2, eps, lr, wd = 0.9, 0.999, 1e-8, 1e-2, 0.01
        m = (1 - b1) * grads
        v = (1 - b2) * grads * grads
        mask = opt.wd_flags.repeat_interleave(128)[: arena.total].float()
        p = start * (1 - lr * wd * mask) - lr * (m / (1 - b1)) / ((v / (1 - b2)).sqrt() + eps)
        dist.all_reduce(p)
        return p / world

    def fused():
        arena.flat_param.copy_(start)
        arena.flat_grad.copy_(grads)
        opt.exp_avg.zero_()
        opt.exp_avg_sq.zero_()
        opt.step_count = 0
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        avg.pending = True
        e0.record()
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    ts = [fused() for _ in range(args.iters)]
    avg.check_status()
    ref = reference()
    err = float((arena.flat_param - ref).abs().max())
    # baseline timing: separate AdamW kernel + NCCL all-reduce + scale
    def baseline():
        arena.flat_param.copy_(start)
        opt.exp_avg.zero_(); opt.exp_avg_sq.zero_(); opt.step_count = 0
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        opt.step()
        dist.all_reduce(arena.flat_param)
        arena.flat_param.mul_(1.0 / world)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    tb = [baseline() for _ in range(args.iters)]
    t = torch.tensor([sorted(ts)[len(ts) // 2], sorted(tb)[len(tb) // 2]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = torch.tensor(1 if err < 1e-5 else 0, device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"world": world, "elems": arena.total, "max_abs_err": err, "ok_all_ranks": bool(int(ok)), "fused_update_avg_ms": round(float(t[0]), 3),
                          "adamw_nccl_scale_ms": round(float(t[1]), 3), "multimem": bool(avg.multicast_ptr)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(ok) else 1)


if __name__ == "__main__":
    main()
