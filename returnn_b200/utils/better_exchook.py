"""
Exception hook that prints the traceback with the whole source statement of every frame (also when it spans several lines) and the
values of the names used in it, follows exception chains (``__cause__`` / ``__context__``), colours its output on a terminal, and can
drop into a debug shell in the failing frame. Own implementation of the idea of returnn/util/better_exchook.py
(better_exchook :1176, format_tb :865, debug_shell :261, dump_all_thread_tracebacks :1355, replace_traceback_format_tb :1582).
"""

from __future__ import annotations
import ast
import io
import keyword
import linecache
import os
import sys
import threading
import tokenize
import traceback
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

_builtin_names = set(dir(__import__("builtins")))


class Color:
    """ANSI colours, switched off when the stream is not a terminal (or by ``CLICOLOR=0`` / ``NO_COLOR``)"""

    codes = {"red": 31, "green": 32, "yellow": 33, "blue": 34, "magenta": 35, "cyan": 36, "bold": 1, "dim": 2}

    def __init__(self, enable: Optional[bool] = None, file=None):
        if enable is None:
            enable = self.is_enabled(file)
        self.enable = bool(enable)

    @staticmethod
    def is_enabled(file=None) -> bool:
        """terminal detection with the usual overrides"""
        if os.environ.get("NO_COLOR") or os.environ.get("CLICOLOR") == "0":
            return False
        if os.environ.get("CLICOLOR_FORCE", "0") not in ("0", ""):
            return True
        file = file or sys.stderr
        try:
            return bool(file.isatty()) and os.environ.get("TERM", "") not in ("", "dumb")
        except Exception:
            return False

    def __call__(self, s: str, color: Optional[str] = None, bold: bool = False) -> str:
        if not self.enable or (color is None and not bold):
            return s
        parts = []
        if bold:
            parts.append("1")
        if color:
            parts.append(str(self.codes[color]))
        return "\x1b[%sm%s\x1b[0m" % (";".join(parts), s)


def _safe_repr(v: Any, limit: int = 300) -> str:
    try:
        if type(v).__module__ in ("torch", "numpy") and hasattr(v, "shape") and hasattr(v, "dtype") and getattr(v, "ndim", 0) > 0:
            s = "<%s shape=%s dtype=%s>" % (type(v).__name__, tuple(v.shape), v.dtype)  # no data dump, no device sync
        else:
            s = repr(v)
    except Exception as e:
        s = "<repr failed: %s: %s>" % (type(e).__name__, e)
    if len(s) > limit:
        s = s[:limit] + "..."
    return s


def get_source_statement(filename: str, lineno: int, module_globals: Optional[Dict[str, Any]] = None) -> Tuple[str, int]:
    """
    The complete statement that contains ``lineno`` (a call spread over several lines is one statement), without the body of a
    compound statement.

    :return: source text (lines joined by newlines, common indentation removed), number of its first line
    """
    lines = linecache.getlines(filename, module_globals)
    if not lines or lineno < 1 or lineno > len(lines):
        return "", lineno
    src = "".join(lines)
    try:
        tree = ast.parse(src, filename)
    except (SyntaxError, ValueError, RecursionError):
        return lines[lineno - 1].strip(), lineno
    best = None
    for node in ast.walk(tree):
        if not isinstance(node, ast.stmt):
            continue
        start, end = node.lineno, getattr(node, "end_lineno", node.lineno)
        body = getattr(node, "body", None)
        if isinstance(body, list) and body and isinstance(body[0], ast.AST):
            end = min(end, max(start, body[0].lineno - 1))  # header of a compound statement only
            # decorators and headers that end on the line of the first body statement (one-liners) stay as they are
            if body[0].lineno == start:
                end = getattr(node, "end_lineno", start)
        if start <= lineno <= end and (best is None or (end - start) < (best[1] - best[0])):
            best = (start, end)
    if best is None:
        return lines[lineno - 1].strip(), lineno
    start, end = best
    end = min(end, start + 14)  # a huge literal is cut
    chunk = [ln.rstrip("\n") for ln in lines[start - 1: end]]
    indent = min((len(ln) - len(ln.lstrip()) for ln in chunk if ln.strip()), default=0)
    return "\n".join(ln[indent:] for ln in chunk), start


def iter_names_in_source(source: str) -> Iterator[str]:
    """dotted names (``a``, ``a.b.c``) in their order of appearance, each once; keywords and attribute-only fragments left out"""
    seen = set()
    try:
        toks = list(tokenize.generate_tokens(io.StringIO(source + "\n").readline))
    except (tokenize.TokenError, IndentationError, SyntaxError):
        toks = []
    i = 0
    while i < len(toks):
        t = toks[i]
        if t.type == tokenize.NAME and not keyword.iskeyword(t.string):
            prev = toks[i - 1] if i else None
            if prev is not None and prev.type == tokenize.OP and prev.string == ".":
                i += 1
                continue  # the tail of an expression like f().attr: no base to look up
            parts = [t.string]
            j = i + 1
            while j + 1 < len(toks) and toks[j].type == tokenize.OP and toks[j].string == "." and toks[j + 1].type == tokenize.NAME:
                parts.append(toks[j + 1].string)
                j += 2
            # a keyword argument name (name=...) is not a variable
            nxt = toks[j] if j < len(toks) else None
            is_kwarg = len(parts) == 1 and nxt is not None and nxt.type == tokenize.OP and nxt.string == "=" and prev is not None and \
                prev.type == tokenize.OP and prev.string in ("(", ",")
            if not is_kwarg:
                for n in range(1, len(parts) + 1):
                    name = ".".join(parts[:n])
                    if name not in seen:
                        seen.add(name)
                        yield name
            i = j
            continue
        i += 1


def _lookup(name: str, f_locals: Dict[str, Any], f_globals: Dict[str, Any]) -> Tuple[bool, Any, str]:
    base, *attrs = name.split(".")
    if base in f_locals:
        v, where = f_locals[base], "local"
    elif base in f_globals:
        v, where = f_globals[base], "global"
    elif base in _builtin_names:
        return False, None, "builtin"
    else:
        return False, None, "not found"
    for a in attrs:
        try:
            v = getattr(v, a)
        except Exception:
            return False, None, "no attribute %r" % a
    return True, v, where


def iter_traceback(tb=None, enforce_most_recent_call_first: bool = False) -> Iterator[Tuple[Any, int]]:
    """
    (frame, line number) pairs of a traceback object, a frame (its stack, outermost first), or a list of
    ``traceback.FrameSummary`` (then the "frame" is the summary).
    """
    if tb is None:
        tb = sys.exc_info()[2]
    items: List[Tuple[Any, int]] = []
    if isinstance(tb, (list, tuple, traceback.StackSummary)):
        items = [(fs, fs.lineno) for fs in tb]
    elif hasattr(tb, "tb_frame"):
        while tb is not None:
            items.append((tb.tb_frame, tb.tb_lineno))
            tb = tb.tb_next
    elif hasattr(tb, "f_back"):
        f = tb
        while f is not None:
            items.append((f, f.f_lineno))
            f = f.f_back
        items.reverse()
    if enforce_most_recent_call_first:
        items.reverse()
    return iter(items)


def format_tb(tb=None, limit: Optional[int] = None, allLocals=None, allGlobals=None, with_vars: bool = True, with_color: Optional[bool] = None,
              file=None) -> List[str]:
    """
    :param tb: traceback, frame or list of frame summaries (default: the exception being handled)
    :param limit: only the innermost ``limit`` frames
    :param allLocals: if a dict is given it is filled with the locals of the innermost frame (for a debug shell); ``allGlobals`` likewise
    :return: lines, each ending in a newline
    """
    color = Color(with_color, file=file)
    out: List[str] = []
    frames = list(iter_traceback(tb))
    skipped = 0
    if limit and len(frames) > limit:
        skipped = len(frames) - limit
        frames = frames[-limit:]
    if skipped:
        out.append(color("  (%i outer frames left out)\n" % skipped, "dim"))
    last_key = None
    repeats = 0
    for f, lineno in frames:
        if hasattr(f, "f_code"):
            co = f.f_code
            filename, funcname, f_locals, f_globals = co.co_filename, co.co_name, f.f_locals, f.f_globals
        else:  # FrameSummary
            filename, funcname, f_locals, f_globals = f.filename, f.name, (f.locals or {}), {}
        key = (filename, lineno, funcname)
        if key == last_key:  # deep recursion: say so once
            repeats += 1
            continue
        if repeats:
            out.append(color("    (the frame above %i more times)\n" % repeats, "dim"))
            repeats = 0
        last_key = key
        out.append("  %s %s, %s %s, %s %s\n" % (color("File", "blue"), color('"%s"' % filename, "cyan"), color("line", "blue"),
                                                color(str(lineno), "magenta"), color("in", "blue"), color(funcname, "yellow", bold=True)))
        source, first = get_source_statement(filename, lineno, f_globals if f_globals else None)
        if not source and not hasattr(f, "f_code") and getattr(f, "line", None):
            source = f.line
        if not source:
            continue
        src_lines = source.split("\n")
        for k, ln in enumerate(src_lines):
            out.append("    %s %s\n" % (color("line:" if k == 0 else "     ", "blue"), ln))
        if with_vars and (f_locals or f_globals):
            out.append("    %s\n" % color("locals:", "blue"))
            for name in iter_names_in_source(source):
                found, v, where = _lookup(name, f_locals, f_globals)
                if not found:
                    if where not in ("builtin",) and "." not in name:
                        out.append("      %s = %s\n" % (color(name, "green"), color("<%s>" % where, "dim")))
                    continue
                if "." not in name and (isinstance(v, type(sys)) or (callable(v) and getattr(v, "__name__", None) == name)):
                    continue  # modules and plain functions / classes under their own name say nothing
                out.append("      %s = %s %s\n" % (color(name, "green"), color("<%s>" % where, "dim"), _safe_repr(v)))
        if allLocals is not None:
            allLocals.clear()
            allLocals.update(f_locals)
        if allGlobals is not None:
            allGlobals.clear()
            allGlobals.update(f_globals)
    if repeats:
        out.append(color("    (the frame above %i more times)\n" % repeats, "dim"))
    return out


def print_tb(tb=None, file=None, **kwargs):
    """:func:`format_tb` written to ``file`` (default stderr)"""
    file = file or sys.stderr
    for line in format_tb(tb, file=file, **kwargs):
        file.write(line)
    file.flush()


def _chain(value: Optional[BaseException]) -> List[Tuple[BaseException, Optional[str]]]:
    """the exception and what led to it, oldest first, with the sentence that joins each to the next"""
    seq: List[Tuple[BaseException, Optional[str]]] = []
    seen = set()
    cur, link = value, None
    while cur is not None and id(cur) not in seen:
        seen.add(id(cur))
        seq.append((cur, link))
        if cur.__cause__ is not None:
            cur, link = cur.__cause__, "The above exception was the direct cause of the following exception:"
        elif cur.__context__ is not None and not cur.__suppress_context__:
            cur, link = cur.__context__, "During handling of the above exception, another exception occurred:"
        else:
            cur = None
    seq.reverse()
    # after the reversal entry i carries the sentence that belongs between entry i and entry i + 1... shift by one
    links = [l for _e, l in seq]
    return [(e, links[i - 1] if i else None) for i, (e, _l) in enumerate(seq)]


def debug_shell(user_ns: Dict[str, Any], user_global_ns: Optional[Dict[str, Any]] = None, traceback=None, execWrapper=None):
    """interactive shell with the given namespace: IPython if importable, else ``code.interact``; nothing on a non-interactive stdin"""
    if not sys.stdin or not sys.stdin.isatty():
        print("debug shell: stdin is not a terminal, skipped", file=sys.stderr)
        return
    ns = dict(user_global_ns or {})
    ns.update(user_ns)
    try:
        import IPython

        IPython.start_ipython(argv=[], user_ns=ns)
        return
    except Exception:
        pass
    import code

    code.interact(banner="debug shell (locals of the failing frame); Ctrl-D to leave", local=ns)


def better_exchook(etype, value, tb, debugshell: bool = False, autodebugshell: bool = True, file=None, with_color: Optional[bool] = None,
                   with_preamble: bool = True):
    """
    ``sys.excepthook`` replacement.

    :param debugshell: open a shell in the failing frame afterwards; ``autodebugshell``: also when the environment says ``DEBUG=1``
    """
    if file is None:
        file = sys.stderr
    color = Color(with_color, file=file)
    all_locals: Dict[str, Any] = {}
    all_globals: Dict[str, Any] = {}
    try:
        if with_preamble:
            print(color("EXCEPTION", "red", bold=True), file=file)
        chain = _chain(value) if isinstance(value, BaseException) else [(value, None)]
        for exc, link in chain:
            if link:
                print("\n%s\n" % link, file=file)
            this_tb = exc.__traceback__ if isinstance(exc, BaseException) and exc is not value else tb
            print(color("Traceback (most recent call last):", "blue"), file=file)
            for line in format_tb(this_tb, allLocals=all_locals, allGlobals=all_globals, with_color=color.enable, file=file):
                file.write(line)
            ename = type(exc).__name__ if isinstance(exc, BaseException) else getattr(etype, "__name__", str(etype))
            msg = str(exc)
            print("%s%s" % (color(ename, "red", bold=True), (": " + msg) if msg else ""), file=file)
            for note in getattr(exc, "__notes__", None) or ():
                print(note, file=file)
    except Exception:
        print("(better_exchook failed itself, standard traceback follows)", file=file)
        traceback.print_exception(etype, value, tb, file=file)
    file.flush()
    if autodebugshell and os.environ.get("DEBUG", "0") not in ("0", ""):
        debugshell = True
    if debugshell:
        debug_shell(all_locals, all_globals, traceback=tb)


def install():
    """install as ``sys.excepthook`` and ``threading.excepthook``"""
    sys.excepthook = better_exchook

    def _thread_hook(args):
        if args.exc_type is SystemExit:
            return
        print("Exception in thread %s:" % (args.thread.name if args.thread else "?"), file=sys.stderr)
        better_exchook(args.exc_type, args.exc_value, args.exc_traceback, autodebugshell=False)

    threading.excepthook = _thread_hook


def setup_all():
    """hook plus the replacement of ``traceback.format_tb`` / ``print_tb`` (loggers and test runners then print the same form)"""
    install()
    replace_traceback_format_tb()
    replace_traceback_print_tb()


def replace_traceback_format_tb():
    """``traceback.format_tb`` and ``StackSummary.format`` give the extended form"""
    traceback.format_tb = lambda tb, limit=None: format_tb(tb, limit=limit, with_color=False)
    if hasattr(traceback, "StackSummary"):
        traceback.StackSummary.format = lambda self, **_kw: format_tb(list(self), with_color=False)


def replace_traceback_print_tb():
    """``traceback.print_tb`` likewise"""
    traceback.print_tb = lambda tb, limit=None, file=None: print_tb(tb, limit=limit, file=file, with_color=False)


def dump_all_thread_tracebacks(exclude_thread_ids: Optional[Sequence[int]] = None, file=None, with_vars: bool = False):
    """stacks of all threads, with their names"""
    if file is None:
        file = sys.stdout
    names = {t.ident: t.name for t in threading.enumerate()}
    for tid, frame in sys._current_frames().items():
        if exclude_thread_ids and tid in exclude_thread_ids:
            continue
        print("Thread %s (%s):" % (tid, names.get(tid, "unknown")), file=file)
        for line in format_tb(frame, with_vars=with_vars, with_color=False):
            file.write(line)
    file.flush()
