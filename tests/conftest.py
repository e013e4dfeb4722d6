"""pytest setup: path, markers, deterministic test environment"""

import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

os.environ.setdefault("RETURNN_TEST", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # the allocation-free entry point test goes last, whatever the file order on the command line
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)
