#!/usr/bin/env python3
"""
Write the raw string stream of a dataset (e.g. ``orth`` / ``raw`` of OggZipDataset or LmDataset) as a Python dict
``{seq_tag: text}``. (reference: tools/dump-dataset-raw-strings.py)
"""

import argparse
import _setup_returnn_env  # noqa: F401
from returnn_b200.datasets.basic import init_dataset


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("dataset", help="dataset dict as a Python expression")
    ap.add_argument("--key", default="raw")
    ap.add_argument("--out", default=None, help="default: stdout")
    ap.add_argument("--epoch", type=int, default=1)
    args = ap.parse_args()
    ds = init_dataset(eval(args.dataset))
    ds.init_seq_order(epoch=args.epoch)
    import contextlib, sys

    with (open(args.out, "w") if args.out else contextlib.nullcontext(sys.stdout)) as out:
        out.write("{\n")
        i = 0
        while ds.is_less_than_num_seqs(i):
            ds.load_seqs(i, i + 1)
            v = ds.get_data(i, args.key)
            text = v.item() if hasattr(v, "item") and getattr(v, "ndim", 1) == 0 else (bytes(v).decode("utf8") if getattr(v, "dtype", None) is not None and v.dtype.kind in "iu" else str(v))
            out.write("%r: %r,\n" % (ds.get_tag(i), text))
            i += 1
        out.write("}\n")


if __name__ == "__main__":
    main()
