#!/usr/bin/env python3
"""
Print the transcriptions of a Bliss corpus, one segment per line (``--with-names``: prefixed by the segment name).
(reference: tools/bliss-dump-text.py)
"""

import argparse
import _setup_returnn_env  # noqa: F401
from _bliss import iter_bliss


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("bliss_filename")
    ap.add_argument("--with-names", action="store_true")
    ap.add_argument("--output", default=None, help="default: stdout")
    args = ap.parse_args()
    import contextlib, sys

    with (open(args.output, "w") if args.output else contextlib.nullcontext(sys.stdout)) as out:
        for item in iter_bliss(args.bliss_filename):
            if item.orth is None:
                continue
            out.write(("%s %s\n" % (item.segment_name, item.orth)) if args.with_names else item.orth + "\n")


if __name__ == "__main__":
    main()
