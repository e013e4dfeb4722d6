#!/usr/bin/env python3
"""
Build the in-tree native libraries (sm_100a CUDA kernels and host helpers) and list their entry points; the reference's
tool of this name compiles one NativeOp from its string source (tools/compile_native_op.py), here all ops live in one library.

    tools/compile_native_op.py [--force] [--ptxas-info]
"""

import argparse
import ctypes
import subprocess
import sys
import _setup_returnn_env  # noqa: F401
from returnn_b200.ops import build


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true")
    args = ap.parse_args()
    for lib in build.build_all(force=args.force, ptxas_info=args.ptxas_info):
        print("built", lib)
        out = subprocess.run(["nm", "-D", "--defined-only", lib], capture_output=True, text=True).stdout
        names = sorted(line.split()[-1] for line in out.splitlines() if " T " in line and "rb200_" in line)
        print("  %i entry points: %s" % (len(names), ", ".join(names)))


if __name__ == "__main__":
    sys.exit(main())
