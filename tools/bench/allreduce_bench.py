"""
Value check and timing of the fused NVLink all-reduce on the GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 \\
        tools/bench/allreduce_bench.py [--elems 100000000] [--no-multimem]

Every rank fills a gradient arena with values that depend on its rank, reduces it bucket by bucket with the fused
kernel, and checks the averaged values and the squared global norm against the closed form; then it times the fused
kernel against ``torch.distributed.all_reduce`` (NCCL) + scale on the same buffer (CUDA events, max over ranks).
Rank 0 prints one JSON line.
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
    ap.add_argument("--elems", type=int, default=100_000_000)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-multimem", action="store_true")
    args = ap.parse_args()
    if args.no_multimem:
        os.environ["RETURNN_B200_ALLREDUCE_MULTIMEM"] = "0"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from returnn_b200.parallel.arena import ParamArena
    from returnn_b200.parallel import fused_allreduce

    # a few "parameters" of odd sizes so that buckets and slices do not fall on round numbers
    sizes = [args.elems // 2 + 3, args.elems // 4 + 1, args.elems // 8 + 130, 7, args.elems // 8]
    params = [(("p%i" % i), torch.nn.Parameter(torch.zeros(s, device=dev))) for i, s in enumerate(sizes)]
    arena = ParamArena(params, bucket_bytes=64 << 20)
    red = fused_allreduce.FusedAllReduce(arena, rank=rank, world=world)
    g = arena.flat_grad
    idx = torch.arange(arena.total, device=dev, dtype=torch.float32)
    base = (idx % 1024) * 1e-3

    def fill():
        g.copy_(base * (rank + 1) + rank)

    # closed form of the average: base * mean(r+1) + mean(r)
    expect = base * (sum(r + 1 for r in range(world)) / world) + sum(range(world)) / world
    fill()
    torch.cuda.synchronize()
    dist.barrier()
    for b, (lo, hi) in enumerate(arena.buckets):
        red.reduce_bucket(b, lo, hi)
    norm_sq = red.finish()
    torch.cuda.synchronize()
    red.check_status()
    err = float((g - expect).abs().max())
    ref_norm = float((expect.double() ** 2).sum())
    norm_err = abs(float(norm_sq) - ref_norm) / ref_norm
    ok = err < 1e-4 and norm_err < 1e-4

    def timed(fn):
        ts = []
        for _ in range(args.iters):
            fill()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor(sorted(ts)[len(ts) // 2], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def run_fused():
        for b, (lo, hi) in enumerate(arena.buckets):
            red.reduce_bucket(b, lo, hi)
        red.finish()

    def run_nccl():
        g.mul_(1.0 / world)
        dist.all_reduce(g)
        torch.linalg.vector_norm(g)

    t_fused = timed(run_fused)
    t_nccl = timed(run_nccl)
    red.check_status()
    # small-vector exchange (batch-norm statistics): value check and latency against NCCL
    small = fused_allreduce.SmallVectorAllReduce(device=dev, rank=rank, world=world)
    vec = torch.arange(1025, device=dev, dtype=torch.float32) * (rank + 1)
    got = small.all_reduce_sum(vec)
    want = torch.arange(1025, device=dev, dtype=torch.float32) * sum(r + 1 for r in range(world))
    small_ok = bool(torch.equal(got, want))
    ok = ok and small_ok
    t_small = timed(lambda: small.all_reduce_sum(vec))
    tmp = vec.clone()
    t_small_nccl = timed(lambda: dist.all_reduce(tmp))
    okt = torch.tensor(1 if ok else 0, device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"small_vector_floats": 1025, "ok": small_ok, "fused_us": round(t_small * 1e3, 1), "nccl_us": round(t_small_nccl * 1e3, 1)}), flush=True)
        nbytes = arena.total * 4
        bus = lambda ms: 2 * (world - 1) / world * nbytes / (ms * 1e-3) / 1e9
        print(json.dumps({"world": world, "elems": arena.total, "multimem": bool(red.multicast_ptr), "max_abs_err": err, "norm_rel_err": norm_err,
                          "ok_all_ranks": bool(int(okt)), "fused_ms": round(t_fused, 3), "nccl_scale_norm_ms": round(t_nccl, 3),
                          "fused_busbw_gbs": round(bus(t_fused), 1), "nccl_busbw_gbs": round(bus(t_nccl), 1)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(okt) else 1)


if __name__ == "__main__":
    main()
