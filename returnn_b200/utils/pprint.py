"""
Pretty printer for config-like Python data: stable, indented, one item per line for containers that do not fit on a
line, numpy arrays summarised, output that is valid Python where the data allows.

Parity: returnn/util/pprint.py (pprint :87, pformat :181).
"""

from __future__ import annotations
from typing import Any
import io
import sys

_MAX_LINE = 100


def _short(obj: Any) -> str:
    try:
        import numpy

        if isinstance(obj, numpy.ndarray):
            if obj.size <= 16:
                return "numpy.array(%r, dtype=%r)" % (obj.tolist(), str(obj.dtype))
            return "<numpy.ndarray shape %s dtype %s>" % (obj.shape, obj.dtype)
        if isinstance(obj, numpy.generic):
            return repr(obj.item())
    except ImportError:
        pass
    return repr(obj)


def _fmt(obj: Any, indent: int, out: io.StringIO):
    pad = " " * indent
    if isinstance(obj, dict) and obj:
        flat = _short(obj) if all(not isinstance(v, (dict, list, tuple, set)) for v in obj.values()) else None
        if flat is not None and len(flat) + indent <= _MAX_LINE:
            out.write(flat)
            return
        out.write("{\n")
        for k, v in obj.items():
            out.write("%s    %r: " % (pad, k))
            _fmt(v, indent + 4, out)
            out.write(",\n")
        out.write(pad + "}")
    elif isinstance(obj, (list, tuple, set)) and obj:
        open_, close_ = {list: "[]", tuple: "()", set: "{}"}[type(obj) if type(obj) in (list, tuple, set) else list]
        items = sorted(obj, key=repr) if isinstance(obj, set) else obj
        flat = open_ + ", ".join(_short(v) for v in items) + ("," if isinstance(obj, tuple) and len(obj) == 1 else "") + close_
        if len(flat) + indent <= _MAX_LINE and all(not isinstance(v, (dict, list, tuple, set)) or not v for v in items):
            out.write(flat)
            return
        out.write(open_ + "\n")
        for v in items:
            out.write(pad + "    ")
            _fmt(v, indent + 4, out)
            out.write(",\n")
        out.write(pad + close_)
    else:
        out.write(_short(obj))


def pformat(obj: Any) -> str:
    """:return: formatted text without trailing newline"""
    out = io.StringIO()
    _fmt(obj, 0, out)
    return out.getvalue()


def pprint(obj: Any, *, file=None, prefix="", postfix="", line_prefix="", line_postfix="\n") -> None:
    """write the formatted object, every line wrapped in ``line_prefix`` / ``line_postfix``"""
    file = file or sys.stdout
    lines = (prefix + pformat(obj) + postfix).split("\n")
    for line in lines:
        file.write(line_prefix + line + line_postfix)
