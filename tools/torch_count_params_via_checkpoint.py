#!/usr/bin/env python3
"""Number of parameters in a checkpoint, per top-level module and in total. (reference: tools/torch_count_params_via_checkpoint.py)"""

import argparse
import collections
import torch
import _setup_returnn_env  # noqa: F401


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("checkpoint")
    ap.add_argument("--depth", type=int, default=1, help="group by this many leading name components")
    args = ap.parse_args()
    model = torch.load(args.checkpoint, map_location="cpu")["model"]
    groups = collections.OrderedDict()
    for k, v in model.items():
        key = ".".join(k.split(".")[: args.depth])
        groups[key] = groups.get(key, 0) + v.numel()
    for k, n in groups.items():
        print("%-50s %12i" % (k, n))
    print("%-50s %12i" % ("total", sum(groups.values())))


if __name__ == "__main__":
    main()
