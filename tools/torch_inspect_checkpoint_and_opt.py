#!/usr/bin/env python3
"""Checkpoint and optimizer state side by side (``torch_inspect_checkpoint.py --opt``). (reference: tools/torch_inspect_checkpoint_and_opt.py)"""

import runpy
import sys
import os

if __name__ == "__main__":
    sys.argv = [sys.argv[0]] + sys.argv[1:] + ["--opt"]
    runpy.run_path(os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_inspect_checkpoint.py"), run_name="__main__")
