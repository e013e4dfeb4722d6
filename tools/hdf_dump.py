#!/usr/bin/env python3
"""
Dump a dataset into a file of the HDF layout (``.hdf`` needs h5py; ``.npz`` works everywhere), reference: tools/hdf_dump.py.

    tools/hdf_dump.py my.config out.npz --dataset train --epoch 1 [--end_seq 1000]
"""

import argparse
import sys
import _setup_returnn_env  # noqa: F401
from returnn_b200.config import Config
from returnn_b200.datasets.basic import init_dataset
from returnn_b200.datasets.hdf import HDFDatasetWriter


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config_or_dataset")
    ap.add_argument("output")
    ap.add_argument("--dataset", default="train")
    ap.add_argument("--epoch", type=int, default=1)
    ap.add_argument("--start_seq", type=int, default=0)
    ap.add_argument("--end_seq", type=int, default=None)
    args = ap.parse_args()
    text = args.config_or_dataset.strip()
    if text.startswith("{"):
        ds_opts = eval(text)
    else:
        cfg = Config()
        cfg.load_file(text)
        ds_opts = cfg.typed_value(args.dataset)
    ds = init_dataset(ds_opts)
    w = HDFDatasetWriter(args.output)
    w.dump_from_dataset(ds, epoch=args.epoch, start_seq=args.start_seq, end_seq=args.end_seq if args.end_seq is not None else float("inf"))
    w.close()
    print("wrote", args.output)


if __name__ == "__main__":
    sys.exit(main())
