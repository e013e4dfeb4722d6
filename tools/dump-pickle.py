#!/usr/bin/env python3
"""Pretty-print a pickle file (or a Python-literal text file). (reference: tools/dump-pickle.py)"""

import argparse
import pickle
import _setup_returnn_env  # noqa: F401
from returnn_b200.utils.pprint import pprint


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("file")
    args = ap.parse_args()
    raw = open(args.file, "rb").read()
    try:
        obj = pickle.loads(raw)
    except Exception:
        from returnn_b200.utils.literal_py_to_pickle import literal_eval

        obj = literal_eval(raw.decode("utf8"))
    pprint(obj)


if __name__ == "__main__":
    main()
