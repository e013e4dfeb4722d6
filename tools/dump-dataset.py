#!/usr/bin/env python3
"""
Print or export the sequences of a dataset given as a config file or a dataset dict string
(reference: tools/dump-dataset.py). Examples:

    tools/dump-dataset.py "{'class': 'Task12AXDataset', 'num_seqs': 5}" --endseq 3
    tools/dump-dataset.py my.config --dataset dev --type stats
"""

import argparse
import sys
import numpy
import _setup_returnn_env  # noqa: F401
from returnn_b200.config import Config
from returnn_b200.datasets.basic import init_dataset
from returnn_b200.log import log


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config_or_dataset")
    ap.add_argument("--dataset", default="train", help="config key of the dataset")
    ap.add_argument("--epoch", type=int, default=1)
    ap.add_argument("--startseq", type=int, default=0)
    ap.add_argument("--endseq", type=int, default=10, help="-1 = all")
    ap.add_argument("--type", default="stdout", choices=["stdout", "null", "stats", "npz"])
    ap.add_argument("--out", default="dump.npz")
    ap.add_argument("--key", default=None, help="only this data key")
    args = ap.parse_args()
    log.initialize(verbosity=[4])
    text = args.config_or_dataset.strip()
    if text.startswith("{"):
        ds_opts = eval(text)
    else:
        cfg = Config()
        cfg.load_file(text)
        ds_opts = cfg.typed_value(args.dataset)
    ds = init_dataset(ds_opts)
    ds.init_seq_order(epoch=args.epoch)
    keys = [args.key] if args.key else ds.get_data_keys()
    stats = {k: [0, 0.0, 0.0, 0] for k in keys}  # frames, sum, sum_sq, seqs
    dump = {}
    i = args.startseq
    while ds.is_less_than_num_seqs(i) and (args.endseq < 0 or i < args.endseq):
        ds.load_seqs(i, i + 1)
        tag = ds.get_tag(i)
        for k in keys:
            d = ds.get_data(i, k)
            if args.type == "stdout":
                with numpy.printoptions(threshold=50, edgeitems=3):
                    print("seq %i tag %r key %r shape %s dtype %s\n%s" % (i, tag, k, d.shape, d.dtype, d))
            elif args.type == "npz":
                dump["%s/%s" % (tag, k)] = d
            if d.dtype.kind in "fiu":
                s = stats[k]
                s[0] += d.shape[0] if d.ndim else 1
                s[1] += float(d.astype("float64").sum())
                s[2] += float((d.astype("float64") ** 2).sum())
                s[3] += 1
        i += 1
    if args.type == "npz":
        numpy.savez(args.out, **dump)
        print("wrote", args.out)
    print("%i sequences" % (i - args.startseq))
    if args.type == "stats":
        for k, (frames, sm, sq, n) in stats.items():
            cnt = max(frames * max(ds.get_data_dim(k) if not ds.is_data_sparse(k) else 1, 1), 1)
            mean = sm / cnt
            print("%s: %i seqs, %i frames, mean %.5f, std %.5f" % (k, n, frames, mean, max(sq / cnt - mean * mean, 0.0) ** 0.5))


if __name__ == "__main__":
    sys.exit(main())
