#!/usr/bin/env python3
"""
Best epoch according to the learning-rate / score file (reference: tools/get-best-model-epoch.py).

    tools/get-best-model-epoch.py my.config [--key dev_loss_ce] [--print_all]
"""

import argparse
import sys
import _setup_returnn_env  # noqa: F401
from returnn_b200.config import Config
from returnn_b200.learning_rate_control import load_learning_rate_control_from_config


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config")
    ap.add_argument("--key", default=None)
    ap.add_argument("--print_all", action="store_true")
    args = ap.parse_args()
    cfg = Config()
    cfg.load_file(args.config)
    lrc = load_learning_rate_control_from_config(cfg)
    scores = []
    for ep, data in sorted(lrc.epoch_data.items()):
        if not data.error:
            continue
        key = args.key or lrc.get_error_key(ep)
        if key in data.error:
            scores.append((data.error[key], ep))
            if args.print_all:
                print("epoch %i: %s = %s (lr %s)" % (ep, key, data.error[key], data.learning_rate))
    if not scores:
        raise SystemExit("no scores found")
    best = min(scores)
    print("best epoch: %i (score %s)" % (best[1], best[0]))


if __name__ == "__main__":
    sys.exit(main())
