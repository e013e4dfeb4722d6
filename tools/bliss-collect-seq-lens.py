#!/usr/bin/env python3
"""
Write ``{segment name: length}`` of a Bliss corpus as a Python dict text file (for ``seq_order_seq_lens_file`` of datasets).
Length = duration * --frame-time-factor (default 100 = 10 ms frames).
(reference: tools/bliss-collect-seq-lens.py)
"""

import argparse
import _setup_returnn_env  # noqa: F401
from _bliss import iter_bliss


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("bliss_filename")
    ap.add_argument("--frame-time-factor", type=float, default=100.0)
    ap.add_argument("--output", default=None, help="default: stdout")
    args = ap.parse_args()
    n = 0
    total = 0.0
    import contextlib, sys

    with (open(args.output, "w") if args.output else contextlib.nullcontext(sys.stdout)) as out:
        out.write("{\n")
        for item in iter_bliss(args.bliss_filename):
            length = max(1, int(round(item.delta_time * args.frame_time_factor)))
            out.write("%r: %i,\n" % (item.segment_name, length))
            n += 1
            total += item.delta_time
        out.write("}\n")
    print("%i segments, %.2f h" % (n, total / 3600.0), file=__import__("sys").stderr)


if __name__ == "__main__":
    main()
