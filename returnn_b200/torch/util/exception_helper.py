"""
Context for an exception inside a step: the batch (tags, shapes, value ranges, invalid labels, sequence lengths) and the
modules on the call stack with their parameter shapes.

Parity: returnn/torch/util/exception_helper.py (help_on_torch_exception :17).
"""

from __future__ import annotations
from typing import Any, List, Optional, Tuple, Union
import sys
import numpy
import torch
from ...log import log
from ...tensor import TensorDict


def _describe(v: Any) -> Tuple[str, Tuple[float, float]]:
    if isinstance(v, torch.Tensor):
        if v.numel() == 0:
            return "shape %s, empty" % (tuple(v.shape),), (0.0, 0.0)
        if v.dtype in (torch.bool,):
            return "shape %s, %s" % (tuple(v.shape), v.dtype), (0.0, 1.0)
        try:
            lo, hi = float(v.min()), float(v.max())
        except Exception as exc:  # e.g. the device is in an error state
            return "shape %s, %s, (min/max unavailable: %s)" % (tuple(v.shape), v.dtype, type(exc).__name__), (0.0, 0.0)
        extra = ""
        if v.is_floating_point():
            extra = ", nan %i, inf %i" % (int(torch.isnan(v).sum()), int(torch.isinf(v).sum()))
        return "shape %s, %s, min/max %g/%g%s" % (tuple(v.shape), v.dtype, lo, hi, extra), (lo, hi)
    if isinstance(v, numpy.ndarray):
        if v.size == 0 or v.dtype.kind in "OUS":
            return "shape %s, %s" % (v.shape, v.dtype), (0.0, 0.0)
        return "shape %s, %s, min/max %g/%g" % (v.shape, v.dtype, v.min(), v.max()), (float(v.min()), float(v.max()))
    return repr(type(v)), (0.0, 0.0)


def help_on_torch_exception(exc: Exception, *, step_idx: Optional[int] = None, extern_data: Optional[TensorDict] = None,
                            model: Union[Any, torch.nn.Module] = None, always_direct_print: bool = False):
    """print what is known about the failing step to the log (and to stderr with ``always_direct_print``)"""
    lines: List[str] = ["%s: %s" % (type(exc).__name__, exc) if exc is not None else "(no exception)", "Step idx: %s" % step_idx]
    if extern_data is not None:
        lines.append("Extern data:")
        if "seq_tag" in extern_data.data:
            lines.append("  Seq tags: %s" % (extern_data.data["seq_tag"].raw_tensor,))
        seen = set()
        for key, data in extern_data.data.items():
            if key == "seq_tag":
                continue
            info, (lo, hi) = _describe(data.raw_tensor)
            lines.append("  %s: %s, %s" % (key, info, data))
            if data.sparse_dim is not None and data.sparse_dim.dimension is not None:
                if lo < 0 or hi >= data.sparse_dim.dimension:
                    lines.append("  WARNING: label outside [0, %i) for sparse dim %s" % (data.sparse_dim.dimension, data.sparse_dim))
            for dim in data.dims:
                if id(dim) in seen or dim.dyn_size_ext is None:
                    continue
                seen.add(id(dim))
                info, _ = _describe(dim.dyn_size_ext.raw_tensor)
                lines.append("    dim %s sizes: %s" % (dim, info))
    # modules on the stack of the exception
    tb = exc.__traceback__ if exc is not None else None
    mods = []
    while tb is not None:
        self_obj = tb.tb_frame.f_locals.get("self")
        if self_obj is not None and (isinstance(self_obj, torch.nn.Module) or type(self_obj).__module__.startswith("returnn_b200.frontend")):
            if hasattr(self_obj, "named_parameters") and not any(m is self_obj for m in mods):
                mods.append(self_obj)
        tb = tb.tb_next
    if mods:
        lines.append("Module call stack:")
        for m in mods:
            try:
                params = ["%s%s" % (n, tuple(p.shape) if hasattr(p, "shape") else tuple(d.dimension for d in p.dims)) for n, p in m.named_parameters(recurse=False)]
            except TypeError:
                params = ["%s" % n for n, _ in m.named_parameters()]
            lines.append("  %s %s" % (type(m).__name__, ", ".join(params)))
    text = "\n".join(lines)
    print(text, file=log.v1)
    if always_direct_print:
        print(text, file=sys.stderr)
