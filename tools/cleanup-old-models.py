#!/usr/bin/env python3
"""
Delete old checkpoints of a training run, keeping the best / last / listed epochs as ``cleanup_old_models`` does during
training (reference: tools/cleanup-old-models.py).

    tools/cleanup-old-models.py --config my.config [--dry_run] [--keep_last_n 3] [--keep_best_n 4]
"""

import argparse
import sys
import _setup_returnn_env  # noqa: F401
from returnn_b200.config import Config, set_global_config
from returnn_b200.log import log
from returnn_b200.engine.base import EngineBase


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", required=True)
    ap.add_argument("--dry_run", action="store_true")
    ap.add_argument("--keep_last_n", type=int, default=None)
    ap.add_argument("--keep_best_n", type=int, default=None)
    args = ap.parse_args()
    cfg = Config()
    cfg.load_file(args.config)
    set_global_config(cfg)
    log.initialize(verbosity=[4])
    opts = cfg.typed_value("cleanup_old_models", None)
    opts = dict(opts) if isinstance(opts, dict) else {}
    if args.keep_last_n is not None:
        opts["keep_last_n"] = args.keep_last_n
    if args.keep_best_n is not None:
        opts["keep_best_n"] = args.keep_best_n
    cfg.set("cleanup_old_models", opts)
    engine = EngineBase(cfg)
    engine.cleanup_old_models(ask_for_confirmation=False, dry_run=args.dry_run) if "dry_run" in engine.cleanup_old_models.__code__.co_varnames else \
        engine.cleanup_old_models(ask_for_confirmation=not args.dry_run)


if __name__ == "__main__":
    sys.exit(main())
