#!/usr/bin/env python3
"""
Print the full segment names of a Bliss corpus, one per line. (reference: tools/bliss-get-segment-names.py)
"""

import argparse
import _setup_returnn_env  # noqa: F401
from _bliss import iter_bliss


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("bliss_filename")
    args = ap.parse_args()
    for item in iter_bliss(args.bliss_filename):
        print(item.segment_name)


if __name__ == "__main__":
    main()
