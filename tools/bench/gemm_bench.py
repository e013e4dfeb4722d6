"""
Micro-benchmark of the tcgen05 GEMM on the linear-layer shapes of the flagship Conformer (forward, data gradient,
weight gradient), against ``torch.matmul`` (cuBLAS) on the same operands.

``python tools/bench/gemm_bench.py [--rows N] [--iters K] [--only NAME]``

Timing: CUDA events on the launching stream, 5 warm-up calls, then ``iters`` calls over a ring of operand sets that
together exceed the L2 capacity, so no call finds its operands cached by the previous one. A spin kernel ahead of the
first event keeps the device busy until the host has queued every launch, so the interval is device time, not launch rate.
"""

from __future__ import annotations
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import argparse
import json
import torch


def _time(fn, n_sets: int, iters: int) -> float:
    for i in range(5):
        fn(i % n_sets)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # keep the GPU busy while the host queues all launches, so that the events bracket device time only
    torch.cuda._sleep(int(2e7 + iters * 1e5))
    e0.record()
    for i in range(iters):
        fn(i % n_sets)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def main():
    from returnn_b200.ops import gemm as G

    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=6656)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--only", default=None)
    ap.add_argument("--wgrad", default="atomic", choices=["atomic", "store"])
    ap.add_argument("--sets", type=int, default=0, help="operand sets in the ring (0: enough to exceed 160 MB)")
    ap.add_argument("--epilogues", action="store_true",
                    help="also time the fused epilogues of the training step on the ff1 / ff2 shapes: bias + SiLU with both outputs + dropout "
                         "(ff1 forward), bias + dropout + half-step residual (ff2 forward), SiLU gradient + dropout mask (ff1 data gradient)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    n = args.rows
    shapes = [("ff1", 512, 2048), ("ff2", 2048, 512), ("qkv", 512, 1536), ("proj", 512, 512), ("pw1", 512, 1024), ("out", 512, 10240)]
    res = []
    for name, din, dout in shapes:
        for kind in ("fwd", "dgrad", "wgrad"):
            tag = "%s_%s" % (name, kind)
            if args.only and args.only != tag:
                continue
            bytes_set = 2 * (n * din + din * dout + n * dout)
            n_sets = args.sets or max(2, int(160e6 // bytes_set) + 1)
            xs = [torch.randn(n, din, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
            ws = [torch.randn(din, dout, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(n_sets)]
            dys = [torch.randn(n, dout, device=dev, dtype=torch.bfloat16) for _ in range(n_sets)]
            if kind == "fwd":
                out = torch.empty(n, dout, device=dev, dtype=torch.bfloat16)
                ours = lambda i: G.gemm(xs[i], ws[i], m=n, n=dout, k=din, a_mn_major=False, b_mn_major=True, out=out)
                ref = lambda i: torch.matmul(xs[i], ws[i], out=out)
            elif kind == "dgrad":
                out = torch.empty(n, din, device=dev, dtype=torch.bfloat16)
                ours = lambda i: G.gemm(dys[i], ws[i], m=n, n=din, k=dout, a_mn_major=False, b_mn_major=False, out=out)
                ref = lambda i: torch.matmul(dys[i], ws[i].t(), out=out)
            else:
                out = torch.empty(din, dout, device=dev, dtype=torch.bfloat16)
                acc = torch.zeros(din, dout, device=dev, dtype=torch.float32)
                if args.wgrad == "atomic":  # dW += X^T dY into an fp32 accumulator, contraction split over CTAs
                    ours = lambda i: G.gemm(xs[i], dys[i], m=din, n=dout, k=n, a_mn_major=True, b_mn_major=True, out=acc, atomic=True)
                else:
                    ours = lambda i: G.gemm(xs[i], dys[i], m=din, n=dout, k=n, a_mn_major=True, b_mn_major=True, out=out)
                ref = lambda i: torch.matmul(xs[i].t(), dys[i], out=out)
            variants = []
            if args.epilogues and name in ("ff1", "ff2") and kind in ("fwd", "dgrad"):
                seed = torch.tensor([1234], dtype=torch.int64, device=dev)
                offs = torch.tensor([0], dtype=torch.int64, device=dev)
                if name == "ff1" and kind == "fwd":
                    bias = torch.randn(dout, device=dev)
                    z = torch.empty(n, dout, device=dev, dtype=torch.bfloat16)
                    variants.append(("bias+silu+z+dropout", lambda i: G.gemm(xs[i], ws[i], m=n, n=dout, k=din, a_mn_major=False, b_mn_major=True, out=z, bias=bias,
                                                                             act="silu", want_act_output=True, out_act=out, dropout_p=0.1, dropout_seed=seed,
                                                                             dropout_offset=offs)))
                    variants.append(("bias+silu", lambda i: G.gemm(xs[i], ws[i], m=n, n=dout, k=din, a_mn_major=False, b_mn_major=True, out=out, bias=bias, act="silu")))
                elif name == "ff2" and kind == "fwd":
                    bias = torch.randn(dout, device=dev)
                    resid = torch.randn(n, dout, device=dev, dtype=torch.bfloat16)
                    variants.append(("bias+dropout+resid", lambda i: G.gemm(xs[i], ws[i], m=n, n=dout, k=din, a_mn_major=False, b_mn_major=True, out=out, bias=bias,
                                                                            dropout_p=0.1, dropout_seed=seed, dropout_offset=offs, resid=resid, res_scale=0.5)))
                elif name == "ff2" and kind == "dgrad":
                    # dX of ff2 is the gradient w.r.t. the activated ff1 output: multiplied by SiLU'(z) and the dropout mask of ff1
                    zz = torch.randn(n, din, device=dev, dtype=torch.bfloat16)
                    variants.append(("dsilu+dropout", lambda i: G.gemm(dys[i], ws[i], m=n, n=din, k=dout, a_mn_major=False, b_mn_major=False, out=out, dact_z=zz,
                                                                       act="silu", dropout_p=0.1, dropout_seed=seed, dropout_offset=offs)))
            for vname, vfn in variants:
                t_v = _time(vfn, n_sets, args.iters)
                print(json.dumps({"shape": tag, "epilogue": vname, "ours_us": round(t_v * 1e6, 2)}), flush=True)
            t_ours = _time(ours, n_sets, args.iters)
            t_ref = _time(ref, n_sets, args.iters)
            flops = 2.0 * n * din * dout
            res.append({"shape": tag, "m_n_k": [n, dout, din], "ours_us": round(t_ours * 1e6, 2), "cublas_us": round(t_ref * 1e6, 2),
                        "ours_tflops": round(flops / t_ours * 1e-12, 1), "cublas_tflops": round(flops / t_ref * 1e-12, 1)})
            print(json.dumps(res[-1]), flush=True)
            del xs, ws, dys
    G.check_status()


if __name__ == "__main__":
    main()
