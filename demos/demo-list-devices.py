#!/usr/bin/env python3
"""Print the CUDA devices PyTorch sees and whether the native sm_100a kernel library is loadable."""

import _setup_env  # noqa: F401
from returnn_b200.torch.util import diagnose_gpu
from returnn_b200.ops import _lib

diagnose_gpu.print_available_devices()
print("native kernel library:", _lib.lib_path(), "loaded" if _lib.get_lib(required=False) is not None else "NOT available")
