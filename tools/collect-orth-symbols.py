#!/usr/bin/env python3
"""
Collect the set of characters that occur in the transcriptions of a corpus (Bliss XML or plain text), with counts.
(reference: tools/collect-orth-symbols.py)
"""

import argparse
import collections
import _setup_returnn_env  # noqa: F401
from returnn_b200.datasets.lm import iter_corpus
from _bliss import iter_bliss


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("filename")
    ap.add_argument("--output", default=None, help="write the symbols as a Python list")
    args = ap.parse_args()
    counts = collections.Counter()
    if ".xml" in args.filename:
        for item in iter_bliss(args.filename):
            counts.update(item.orth or "")
    else:
        iter_corpus(args.filename, lambda line: counts.update(line))
    for ch, c in sorted(counts.items()):
        print("%r %i" % (ch, c))
    if args.output:
        with open(args.output, "w") as f:
            f.write(repr(sorted(counts.keys())) + "\n")


if __name__ == "__main__":
    main()
