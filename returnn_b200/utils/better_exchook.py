"""
Exception hook that prints the traceback with the source lines and the values of the local variables used on them.
Own compact implementation of the idea of returnn/util/better_exchook.py.
"""

from __future__ import annotations
import sys
import linecache
import re
import threading
import traceback

_ident_re = re.compile(r"[A-Za-z_][A-Za-z0-9_]*(?:\.[A-Za-z_][A-Za-z0-9_]*)*")
_keywords = {"None", "True", "False", "and", "or", "not", "in", "is", "if", "else", "for", "while", "return", "def", "class",
             "import", "from", "as", "with", "lambda", "yield", "assert", "raise", "try", "except", "finally", "pass", "self"}


def _safe_repr(v, limit: int = 120) -> str:
    try:
        s = repr(v)
    except Exception as e:
        s = "<repr failed: %s>" % e
    if len(s) > limit:
        s = s[:limit] + "..."
    return s


def format_tb(tb=None, limit=None, allLocals=None, allGlobals=None, with_vars: bool = True):
    """list of formatted lines for a traceback (or a stack frame list)"""
    out = []
    frames = []
    if tb is None:
        tb = sys.exc_info()[2]
    while tb is not None:
        frames.append((tb.tb_frame, tb.tb_lineno))
        tb = tb.tb_next
    if limit:
        frames = frames[-limit:]
    for f, lineno in frames:
        co = f.f_code
        out.append('  File "%s", line %i, in %s\n' % (co.co_filename, lineno, co.co_name))
        line = linecache.getline(co.co_filename, lineno, f.f_globals).strip()
        if line:
            out.append("    line: %s\n" % line)
            if with_vars:
                seen = set()
                for m in _ident_re.finditer(line):
                    name = m.group(0)
                    base = name.split(".")[0]
                    if base in _keywords or name in seen:
                        continue
                    seen.add(name)
                    scope = f.f_locals if base in f.f_locals else (f.f_globals if base in f.f_globals else None)
                    if scope is None:
                        continue
                    try:
                        v = scope[base]
                        for part in name.split(".")[1:]:
                            v = getattr(v, part)
                    except Exception:
                        continue
                    if callable(v) and not isinstance(v, type) and hasattr(v, "__name__"):
                        continue
                    out.append("      %s = %s\n" % (name, _safe_repr(v)))
    return out


def better_exchook(etype, value, tb, debugshell=False, autodebugshell=True, file=None, with_color=None, with_preamble=True):
    """sys.excepthook replacement"""
    if file is None:
        file = sys.stderr
    try:
        if with_preamble:
            print("EXCEPTION", file=file)
            print("Traceback (most recent call last):", file=file)
        for line in format_tb(tb):
            file.write(line)
        print("%s: %s" % (getattr(etype, "__name__", etype), value), file=file)
    except Exception:
        traceback.print_exception(etype, value, tb, file=file)
    file.flush()


def install():
    """install as sys.excepthook and threading.excepthook"""
    sys.excepthook = better_exchook

    def _thread_hook(args):
        better_exchook(args.exc_type, args.exc_value, args.exc_traceback)

    threading.excepthook = _thread_hook


def dump_all_thread_tracebacks(exclude_thread_ids=None, file=None):
    """stacks of all threads"""
    if file is None:
        file = sys.stdout
    frames = sys._current_frames()
    for tid, frame in frames.items():
        if exclude_thread_ids and tid in exclude_thread_ids:
            continue
        print("Thread %s:" % tid, file=file)
        for line in traceback.format_stack(frame):
            file.write(line)
