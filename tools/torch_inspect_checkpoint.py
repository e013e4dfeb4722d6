#!/usr/bin/env python3
"""
List the contents of a checkpoint (``<model>.NNN.pt``) and optionally of the optimizer file next to it
(reference: tools/torch_inspect_checkpoint.py, torch_inspect_checkpoint_and_opt.py, torch_count_params_via_checkpoint.py).

    tools/torch_inspect_checkpoint.py model.010.pt [--key layers.0.weight] [--opt] [--stats]
"""

import argparse
import os
import sys
import torch
import _setup_returnn_env  # noqa: F401


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("checkpoint")
    ap.add_argument("--key", default=None, help="print this tensor")
    ap.add_argument("--opt", action="store_true", help="also inspect <checkpoint without .pt>.opt.pt")
    ap.add_argument("--stats", action="store_true", help="mean / std / min / max per tensor")
    args = ap.parse_args()
    ck = torch.load(args.checkpoint, map_location="cpu")
    print("epoch:", ck.get("epoch"), "step:", ck.get("step"), "other keys:", [k for k in ck if k not in ("model", "epoch", "step")])
    model = ck["model"]
    total = 0
    for k, v in model.items():
        total += v.numel()
        line = "%-70s %-20s %s" % (k, tuple(v.shape), str(v.dtype).replace("torch.", ""))
        if args.stats and v.is_floating_point() and v.numel():
            f = v.float()
            line += "  mean %.4g std %.4g min %.4g max %.4g" % (f.mean(), f.std() if f.numel() > 1 else 0.0, f.min(), f.max())
        print(line)
    print("parameters: %i tensors, %i values (%.1f M)" % (len(model), total, total / 1e6))
    if args.key:
        print(args.key, model[args.key])
    if args.opt:
        fn = args.checkpoint[:-3] + ".opt.pt" if args.checkpoint.endswith(".pt") else args.checkpoint + ".opt.pt"
        if not os.path.exists(fn):
            print("no optimizer file", fn)
            return
        opt = torch.load(fn, map_location="cpu")
        sd = opt.get("optimizer", opt)
        print("optimizer param groups:", [{k: v for k, v in g.items() if k != "params"} for g in sd["param_groups"]])
        names = opt.get("param_names")
        for idx, st in list(sd["state"].items())[:10]:
            print(names[idx] if names else idx, {k: (tuple(v.shape) if hasattr(v, "shape") else v) for k, v in st.items()})


if __name__ == "__main__":
    sys.exit(main())
