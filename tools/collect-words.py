#!/usr/bin/env python3
"""
Count the words of a text file or Bliss corpus and print them by frequency (``--vocab-out``: write a vocabulary dict).
(reference: tools/collect-words.py)
"""

import argparse
import collections
import _setup_returnn_env  # noqa: F401
from returnn_b200.datasets.lm import iter_corpus
from _bliss import iter_bliss


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("filename")
    ap.add_argument("--type", choices=["text", "bliss"], default=None)
    ap.add_argument("--vocab-out", default=None)
    ap.add_argument("--min-count", type=int, default=1)
    args = ap.parse_args()
    kind = args.type or ("bliss" if ".xml" in args.filename else "text")
    counts = collections.Counter()
    if kind == "bliss":
        for item in iter_bliss(args.filename):
            counts.update((item.orth or "").split())
    else:
        iter_corpus(args.filename, lambda line: counts.update(line.split()))
    words = [(w, c) for w, c in counts.most_common() if c >= args.min_count]
    for w, c in words:
        print("%s %i" % (w, c))
    if args.vocab_out:
        with open(args.vocab_out, "w") as f:
            f.write("{\n" + "".join("%r: %i,\n" % (w, i) for i, (w, _) in enumerate(words)) + "}\n")


if __name__ == "__main__":
    main()
