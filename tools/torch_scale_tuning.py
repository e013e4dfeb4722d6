#!/usr/bin/env python3
"""
Grid search over log-linear score combination weights: given per-hypothesis scores of several models (an n-best list as a
Python dict ``{seq_tag: [(hyp text, {score name: value})...]}``) and references (``{seq_tag: text}``), find the scales that
minimise the word error rate of the 1-best. (reference: tools/torch_scale_tuning.py)
"""

import argparse
import itertools
import _setup_returnn_env  # noqa: F401


def _edit_distance(a, b):
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("nbest", help="Python dict file")
    ap.add_argument("refs", help="Python dict file")
    ap.add_argument("--scales", default="0,0.1,0.2,0.3,0.5,0.7,1.0", help="candidate values per score (the first score is fixed to 1)")
    args = ap.parse_args()
    nbest = eval(open(args.nbest).read())
    refs = eval(open(args.refs).read())
    names = sorted({k for hyps in nbest.values() for _, sc in hyps for k in sc})
    cands = [float(x) for x in args.scales.split(",")]
    total_ref = sum(len(refs[t].split()) for t in nbest)
    best = None
    for combo in itertools.product(*([[1.0]] + [cands] * (len(names) - 1))):
        errs = 0
        for tag, hyps in nbest.items():
            hyp = max(hyps, key=lambda h: sum(s * h[1].get(n, 0.0) for s, n in zip(combo, names)))[0]
            errs += _edit_distance(hyp.split(), refs[tag].split())
        wer = errs / max(total_ref, 1)
        if best is None or wer < best[0]:
            best = (wer, combo)
    print("scores:", names)
    print("best scales:", dict(zip(names, best[1])), "WER %.2f%%" % (100 * best[0]))


if __name__ == "__main__":
    main()
