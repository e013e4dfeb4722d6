"""
Find the first operation that produces an inf or nan: run a function under a dispatch mode that inspects the output of
every ATen op and prints the op with the Python stack (up to the caller of :func:`debug_inf_nan`).

Parity: returnn/torch/util/debug_inf_nan.py (debug_inf_nan :50, _TraceOps :120).
"""

from __future__ import annotations
from typing import Callable, Optional, TextIO
import sys
import traceback
import torch
from torch.utils._python_dispatch import TorchDispatchMode

# ops whose non-finite outputs are intended or uninformative (allocations, masks with -inf, views)
_IGNORED = {
    "aten::empty.memory_format", "aten::zeros_like", "aten::ones_like", "aten::full", "aten::scalar_tensor", "aten::_local_scalar_dense",
    "aten::where.self", "aten::detach", "aten::_to_copy", "aten::clone", "aten::stack", "aten::view", "aten::_unsafe_view", "aten::permute",
    "aten::t", "aten::split_with_sizes", "aten::slice.Tensor", "aten::select.int", "aten::masked_fill.Scalar", "aten::masked_fill_.Scalar",
    "aten::full_like", "aten::fill_.Scalar", "aten::max_pool2d_with_indices",
}


class _Inspect(TorchDispatchMode):
    def __init__(self, *, depth_base: int, file: TextIO, report_every_op_call: bool, stop_after_first: bool):
        super().__init__()
        self.depth_base = depth_base
        self.file = file
        self.report_every_op_call = report_every_op_call
        self.stop_after_first = stop_after_first
        self.found = False

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        if self.found and self.stop_after_first:
            return out
        name = func._schema.name + ("." + func._schema.overload_name if func._schema.overload_name else "")
        if name in _IGNORED:
            return out
        if self.report_every_op_call:
            print("--- op %s" % name, file=self.file)
        outs = out if isinstance(out, (tuple, list)) else [out]
        for i, t in enumerate(outs):
            if not isinstance(t, torch.Tensor) or not (t.is_floating_point() or t.is_complex()) or t.numel() == 0:
                continue
            n_nan = int(torch.isnan(t).sum())
            n_inf = int(torch.isinf(t).sum())
            if n_nan or n_inf:
                self.found = True
                print("op %s output %i (shape %s, %s): %i nan, %i inf of %i" % (name, i, tuple(t.shape), t.dtype, n_nan, n_inf, t.numel()),
                      file=self.file)
                stack = traceback.extract_stack()[self.depth_base: -1]
                stack = [fr for fr in stack if "/torch/" not in fr.filename.replace("\\", "/") or "returnn" in fr.filename]
                for line in traceback.format_list(stack[-12:]):
                    print(line.rstrip(), file=self.file)
                break
        return out


def debug_inf_nan(func: Callable[[], Optional[torch.Tensor]], *, with_grad: bool = False, report_every_op_call: bool = True,
                  stop_reporting_after_first_inf_nan: bool = True, file: Optional[TextIO] = None):
    """
    :param func: called without arguments; with ``with_grad`` it returns the loss and ``loss.backward()`` runs under anomaly detection
    :param report_every_op_call: print every op (a trace up to the failure)
    :param stop_reporting_after_first_inf_nan: report only the first offender
    :param file: default stdout
    """
    file = file or sys.stdout
    depth = len(traceback.extract_stack()) - 1
    mode = _Inspect(depth_base=depth, file=file, report_every_op_call=report_every_op_call, stop_after_first=stop_reporting_after_first_inf_nan)
    if not with_grad:
        with mode:
            func()
        return
    with torch.autograd.detect_anomaly():
        with mode:
            loss = func()
        file.flush()
        try:
            loss.backward()
        except RuntimeError as exc:
            print("RuntimeError in backward: %s" % exc, file=file)
