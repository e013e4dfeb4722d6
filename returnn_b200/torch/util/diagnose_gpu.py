"""
GPU diagnostics: device reports at startup, hints when no GPU is found, a watchdog for calls that may hang
(``torch.cuda.is_available()`` on a broken driver), memory cleanup helpers.

Parity: returnn/torch/util/diagnose_gpu.py:21-210.
"""

from __future__ import annotations
from typing import List, Optional
import gc
import os
import subprocess
import sys
import torch


def print_available_devices(*, file=None):
    """one line per CUDA device"""
    if file is None:
        file = sys.stdout
    print("CUDA_VISIBLE_DEVICES=%s" % os.environ.get("CUDA_VISIBLE_DEVICES", "<unset>"), file=file)
    if not torch.cuda.is_available():
        print("(CUDA not available)", file=file)
        return
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        print("  %i: %s, sm_%i%i, %.0f GB, %i SMs" % (i, p.name, p.major, p.minor, p.total_memory / 2 ** 30, p.multi_processor_count), file=file)


def print_using_cuda_device_report(dev, *, file=None):
    """details for the device in use"""
    if file is None:
        file = sys.stdout
    dev = torch.device(dev)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    p = torch.cuda.get_device_properties(idx)
    free, total = torch.cuda.mem_get_info(idx)
    print("Using gpu device %i: %s (sm_%i%i), %.1f GB free of %.1f GB" % (idx, p.name, p.major, p.minor, free / 2 ** 30, total / 2 ** 30), file=file)


def diagnose_no_gpu() -> List[str]:
    """hints when CUDA is requested but not available"""
    res = ["torch.cuda.is_available() is False; torch %s built for CUDA %s" % (torch.__version__, torch.version.cuda)]
    res.append("CUDA_VISIBLE_DEVICES=%s" % os.environ.get("CUDA_VISIBLE_DEVICES", "<unset>"))
    try:
        out = subprocess.check_output(["nvidia-smi", "-L"], stderr=subprocess.STDOUT, timeout=10).decode()
        res.append("nvidia-smi -L:\n" + out.strip())
    except Exception as exc:
        res.append("nvidia-smi failed: %s" % exc)
    return res


def garbage_collect():
    """Python GC + CUDA cache"""
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def timeout(func_expr: str = "torch.cuda.is_available()", *, timeout_sec: float = 30.0) -> Optional[str]:
    """
    Evaluate an expression in a subprocess with a time limit. Used before the first CUDA call of the main process:
    a hanging driver then costs 30 seconds instead of the job.

    :return: stdout of the subprocess, or None on timeout / failure
    """
    code = "import torch; print(%s)" % func_expr
    try:
        out = subprocess.check_output([sys.executable, "-c", code], timeout=timeout_sec, stderr=subprocess.DEVNULL)
        return out.decode().strip()
    except subprocess.TimeoutExpired:
        print("diagnose_gpu: %r did not return within %.0f s" % (func_expr, timeout_sec), file=sys.stderr)
        return None
    except Exception:
        return None


def print_relevant_env_vars(*, file=None):
    """the environment variables that decide which devices a process sees and how the CUDA libraries behave"""
    import os
    import sys

    file = file or sys.stdout
    names = sorted(k for k in os.environ if k.startswith(("CUDA", "NCCL", "TORCH_", "PYTORCH_", "RETURNN_B200_", "NVIDIA_", "OMP_NUM", "LD_LIBRARY")))
    for k in names:
        print("%s=%s" % (k, os.environ[k]), file=file)
    if not names:
        print("(none of the CUDA / NCCL / torch variables is set)", file=file)
