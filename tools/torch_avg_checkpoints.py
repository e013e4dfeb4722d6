#!/usr/bin/env python3
"""
Average the model parameters of several checkpoints (reference: tools/torch_avg_checkpoints.py).

    tools/torch_avg_checkpoints.py --checkpoints model.010.pt model.011.pt model.012.pt --output_path model.avg.pt
    tools/torch_avg_checkpoints.py --prefix model. --postfix .pt --epochs 10,11,12 --output_path model.avg.pt
"""

import argparse
import sys
import torch
import _setup_returnn_env  # noqa: F401


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoints", nargs="*", default=[])
    ap.add_argument("--prefix", default=None)
    ap.add_argument("--postfix", default=".pt")
    ap.add_argument("--epochs", default=None, help="comma separated, with --prefix")
    ap.add_argument("--output_path", required=True)
    args = ap.parse_args()
    files = list(args.checkpoints)
    if args.prefix and args.epochs:
        files += ["%s%03d%s" % (args.prefix, int(e), args.postfix) for e in args.epochs.split(",")]
    assert files, "no checkpoints given"
    avg, first = None, None
    for fn in files:
        ck = torch.load(fn, map_location="cpu")
        model = ck["model"]
        if avg is None:
            first = ck
            avg = {k: v.clone().double() if v.is_floating_point() else v.clone() for k, v in model.items()}
        else:
            assert set(model.keys()) == set(avg.keys()), "%s has different parameters" % fn
            for k, v in model.items():
                if v.is_floating_point():
                    avg[k] += v.double()
        print("read", fn, "epoch", ck.get("epoch"), "step", ck.get("step"))
    n = len(files)
    out = {k: (v / n).to(first["model"][k].dtype) if v.is_floating_point() else v for k, v in avg.items()}
    result = dict(first)
    result["model"] = out
    result["averaged_from"] = files
    torch.save(result, args.output_path)
    print("wrote", args.output_path)


if __name__ == "__main__":
    sys.exit(main())
