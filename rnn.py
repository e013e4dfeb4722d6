#!/usr/bin/env python3
"""
Main entry point: ``rnn.py <config> [++key value ...]``.

Configs written for RETURNN (``import returnn.frontend as rf``) run unchanged: the ``returnn`` import name is aliased to
this package before the config is loaded.
"""

import os
import sys

_my_dir = os.path.dirname(os.path.abspath(__file__))
if _my_dir not in sys.path:
    sys.path.insert(0, _my_dir)

import returnn_b200  # noqa: E402

returnn_b200.install_returnn_alias()

from returnn_b200.__main__ import main  # noqa: E402

if __name__ == "__main__":
    main(sys.argv)
