#!/usr/bin/env python3
"""
Convert parallel text files (source / target, one sentence per line) plus vocabularies into the dataset file layout
(``data`` = source ids, ``classes`` = target ids). Writes ``.npz`` (always available) or HDF (with h5py).
(reference: tools/hdf_dump_translation_dataset.py)
"""

import argparse
import numpy
import _setup_returnn_env  # noqa: F401
from returnn_b200.datasets.hdf import NpzWriter, SimpleHDFWriter


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--source", required=True)
    ap.add_argument("--target", required=True)
    ap.add_argument("--source-vocab", required=True, help="Python dict {token: id}")
    ap.add_argument("--target-vocab", required=True)
    ap.add_argument("--unk", default="<unk>")
    ap.add_argument("--output", required=True)
    args = ap.parse_args()
    sv, tv = eval(open(args.source_vocab).read()), eval(open(args.target_vocab).read())
    writer_cls = SimpleHDFWriter if args.output.endswith(".hdf") else NpzWriter
    writer = writer_cls(args.output, dim=len(sv), ndim=1, extra_type={"classes": (len(tv), 1, "int32")})
    n = 0
    with open(args.source, encoding="utf8") as fs, open(args.target, encoding="utf8") as ft:
        for i, (s, t) in enumerate(zip(fs, ft)):
            src = numpy.array([sv.get(w, sv.get(args.unk, 0)) for w in s.split()], dtype="int32")
            tgt = numpy.array([tv.get(w, tv.get(args.unk, 0)) for w in t.split()], dtype="int32")
            if not len(src) or not len(tgt):
                continue
            writer.insert_batch(src[None], [len(src)], ["line-%i" % i], extra={"classes": tgt[None]})
            n += 1
    writer.close()
    print("wrote %i sentence pairs to %s" % (n, args.output))


if __name__ == "__main__":
    main()
