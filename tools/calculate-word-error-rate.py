#!/usr/bin/env python3
"""
Word error rate between two files that hold a Python dict ``{seq_tag: "text"}`` each (as written by the search /
forward tasks), reference: tools/calculate-word-error-rate.py.

    tools/calculate-word-error-rate.py --hyps hyp.py --refs ref.py [--expect_full] [--out wer.txt]
"""

import argparse
import gzip
import sys
import _setup_returnn_env  # noqa: F401
from returnn_b200.utils.literal_py_to_pickle import literal_eval


def _load(fn):
    raw = (gzip.open(fn, "rb") if fn.endswith(".gz") else open(fn, "rb")).read()
    d = literal_eval(raw)
    assert isinstance(d, dict), "%s: expected a dict" % fn
    return d


def edit_ops(ref, hyp):
    """(substitutions, deletions, insertions) of the best alignment"""
    n, m = len(ref), len(hyp)
    cost = [[(j, 0, 0, j) for j in range(m + 1)]] + [[(i, 0, i, 0)] + [None] * m for i in range(1, n + 1)]
    for i in range(1, n + 1):
        for j in range(1, m + 1):
            c_sub = cost[i - 1][j - 1]
            sub = (c_sub[0] + (ref[i - 1] != hyp[j - 1]), c_sub[1] + (ref[i - 1] != hyp[j - 1]), c_sub[2], c_sub[3])
            c_del = cost[i - 1][j]
            dele = (c_del[0] + 1, c_del[1], c_del[2] + 1, c_del[3])
            c_ins = cost[i][j - 1]
            ins = (c_ins[0] + 1, c_ins[1], c_ins[2], c_ins[3] + 1)
            cost[i][j] = min(sub, dele, ins)
    return cost[n][m][1:]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hyps", required=True)
    ap.add_argument("--refs", required=True)
    ap.add_argument("--expect_full", action="store_true", help="every reference must have a hypothesis")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    hyps, refs = _load(args.hyps), _load(args.refs)
    S = D = I = N = 0
    missing = 0
    for tag, ref in refs.items():
        if tag not in hyps:
            missing += 1
            if args.expect_full:
                raise SystemExit("no hypothesis for %r" % tag)
            continue
        hyp = hyps[tag]
        if isinstance(hyp, (list, tuple)):  # n-best list of (score, text): take the best
            hyp = max(hyp)[1] if hyp and isinstance(hyp[0], (list, tuple)) else " ".join(hyp)
        s, d, i = edit_ops(ref.split(), hyp.split())
        S, D, I, N = S + s, D + d, I + i, N + len(ref.split())
    wer = 100.0 * (S + D + I) / max(N, 1)
    print("seqs: %i (missing hyps: %i), ref words: %i, sub %i del %i ins %i" % (len(refs), missing, N, S, D, I))
    print("WER: %.2f%%" % wer)
    if args.out:
        with open(args.out, "w") as f:
            f.write("%f\n" % wer)


if __name__ == "__main__":
    sys.exit(main())
