"""
Logging: five verbosity streams ``log.v1`` .. ``log.v5`` (``print(..., file=log.v3)``), fanned out to several sinks
(``stdout``, files), each sink with its own verbosity and format. Under distributed training each rank's file sink
gets the suffix ``.torch-distrib-<rank>-<size>``.

Parity: returnn/log.py (Log.initialize :74, init_by_config :176-208).
"""

from __future__ import annotations
from typing import List, Optional, Sequence, Union
import io
import logging
import os
import sys
import threading
import contextlib
import time


class Stream:
    """File-like object that forwards complete lines to a :class:`logging.Logger` at a fixed level."""

    def __init__(self, log: logging.Logger, lvl: int):
        self.buf = io.StringIO()
        self.log = log
        self.lvl = lvl
        self.lock = threading.RLock()

    def write(self, msg: str):
        """buffer until flush/newline"""
        with self.lock:
            if msg == "\n":
                self.flush()
            else:
                self.buf.write(msg)
                if msg.endswith("\n"):
                    self.flush()

    def flush(self):
        """emit the buffer"""
        with self.lock:
            self.buf.flush()
            s = self.buf.getvalue()
            if s.endswith("\n"):
                s = s[:-1]
            if s:
                self.log.log(self.lvl, s)
            self.buf.seek(0)
            self.buf.truncate(0)

    def isatty(self):
        """never"""
        return False


class _NullStream:
    def write(self, msg):
        pass

    def flush(self):
        pass


class Log:
    """
    ``log.v[i]`` / ``log.v1``..``log.v5`` are streams; ``log.verbose[i]`` says whether level i is shown anywhere.
    Before :func:`initialize`, everything up to level 3 goes to stdout.
    """

    def __init__(self):
        self.initialized = False
        self.filename: Optional[str] = None
        self.v: List = []
        self.verbose: List[bool] = [False] * 6
        self._loggers: List[logging.Logger] = []
        self._printed_warning_history = set()
        self.initialize(verbosity=[3], _initial=True)

    def initialize(
        self,
        logs: Optional[Sequence[str]] = None,
        verbosity: Optional[Sequence[int]] = None,
        formatter: Optional[Sequence[str]] = None,
        propagate: bool = False,
        _initial: bool = False,
    ):
        """
        :param logs: sink names: "stdout", "|<cmd>" is not supported, anything else is a filename
        :param verbosity: one verbosity (0..5) per sink; a single value applies to all
        :param formatter: "default", "timed", "raw" or "verbose" per sink
        """
        logs = list(logs) if logs else []
        verbosity = list(verbosity) if verbosity else []
        formatter = list(formatter) if formatter else []
        fmt = {
            "default": logging.Formatter("%(message)s"),
            "timed": logging.Formatter("%(asctime)s %(message)s", datefmt="%Y-%m-%d,%H:%M:%S.%MS"),
            "raw": logging.Formatter("%(message)s"),
            "verbose": logging.Formatter("%(levelname)s - %(asctime)s %(message)s", datefmt="%Y-%m-%d,%H:%M:%S.%MS"),
        }
        for lg in self._loggers:
            for h in list(lg.handlers):
                lg.removeHandler(h)
                if isinstance(h, logging.FileHandler):
                    h.close()
        self._loggers = [logging.getLogger("returnn_b200.v" + str(v)) for v in range(6)]
        for lg in self._loggers:
            lg.setLevel(logging.DEBUG)
            lg.propagate = propagate
            lg.handlers = []
        if "stdout" not in logs and not any(x in ("stdout", "stderr") for x in logs):
            logs.append("stdout")
        if len(verbosity) == 1 and len(logs) > 1:
            verbosity = verbosity * len(logs)
        elif len(verbosity) < len(logs):
            verbosity = verbosity + [verbosity[-1] if verbosity else 3] * (len(logs) - len(verbosity))
        if len(formatter) == 1 and len(logs) > 1:
            formatter = formatter * len(logs)
        self.verbose = [False] * 6
        self.filename = None
        for i, t in enumerate(logs):
            vlevel = int(verbosity[i])
            assert 0 <= vlevel <= 5, "invalid verbosity: %r" % (verbosity[i],)
            f = fmt["default"] if i >= len(formatter) or not formatter[i] else fmt[formatter[i]]
            if t == "stdout":
                handler = _StdoutHandler()
            elif t == "stderr":
                handler = logging.StreamHandler(sys.stderr)
            elif t.startswith("|"):
                raise ValueError("log sink %r: pipes into commands are not supported" % t)
            else:
                d = os.path.dirname(t)
                if d:
                    os.makedirs(d, exist_ok=True)
                if self.filename is None:
                    self.filename = t
                handler = logging.FileHandler(t)
            handler.setLevel(logging.DEBUG)
            handler.setFormatter(f)
            for j in range(vlevel + 1):
                self.verbose[j] = True
                self._loggers[j].addHandler(handler)
        null = _NullStream()
        self.v = [Stream(self._loggers[j], logging.DEBUG) if self.verbose[j] else null for j in range(6)]
        self.error = self.v[0]
        self.v0, self.v1, self.v2, self.v3, self.v4, self.v5 = self.v
        self.initialized = not _initial

    def init_by_config(self, config):
        """
        Reads ``log``, ``log_verbosity``, ``log_format``.

        :param returnn_b200.config.Config config:
        """
        logs = config.list("log", [])
        log_verbosity = config.int_list("log_verbosity", [])
        log_format = config.list("log_format", [])
        if config.typed_value("torch_distributed") is not None:
            from returnn_b200.torch import distributed as _dist

            ctx = _dist.get_ctx(config=config)
            if ctx is not None:
                suffix = ".torch-distrib-%i-%i" % (ctx.rank(), ctx.size())
                new_logs = []
                for fn in logs:
                    if fn in ("stdout", "stderr") or fn.startswith("|"):
                        new_logs.append(fn)
                    else:
                        fn_prefix, fn_ext = os.path.splitext(fn)
                        new_logs.append(fn_prefix + suffix + fn_ext)
                logs = new_logs
        self.initialize(logs=logs, verbosity=log_verbosity or [3], formatter=log_format)

    def print_warning(self, text: str, prefix_text: str = "WARNING:", extra_text: Optional[str] = None):
        """print a warning once per distinct text"""
        if text in self._printed_warning_history:
            return
        self._printed_warning_history.add(text)
        print(prefix_text, text, file=self.v2)
        if extra_text:
            print(extra_text, file=self.v2)

    def print_deprecation_warning(self, text: str, behavior_version: Optional[int] = None):
        """deprecation warning; an error once the behavior version reached the given one"""
        if behavior_version is not None:
            from .utils.basic import BehaviorVersion

            BehaviorVersion.require(False, text, behavior_version)
        self.print_warning(text, prefix_text="DEPRECATION WARNING:")

    def flush(self):
        """flush all streams"""
        for s in self.v:
            s.flush()


class _StdoutHandler(logging.StreamHandler):
    """Always writes to the *current* ``sys.stdout`` (pytest capture, redirections)."""

    def __init__(self):
        super().__init__(sys.stdout)

    def emit(self, record):
        self.stream = sys.stdout
        super().emit(record)


log = Log()


class StreamThreadLocal(threading.local):
    """per-thread StringIO, used by :class:`StreamDummy`-style capture"""

    def __init__(self):
        self.buf = io.StringIO()


@contextlib.contextmanager
def wrap_log_streams(alt_stream, also_sys_stdout: bool = False, tmp_replace_attribs=("v", "v1", "v2", "v3", "v4", "v5", "error")):
    """temporarily send all log streams to alt_stream"""
    old = {k: getattr(log, k) for k in tmp_replace_attribs}
    old_stdout = sys.stdout
    log.v = [alt_stream] * 6
    for k in tmp_replace_attribs:
        if k != "v":
            setattr(log, k, alt_stream)
    if also_sys_stdout:
        sys.stdout = alt_stream
    try:
        yield
    finally:
        for k, v in old.items():
            setattr(log, k, v)
        sys.stdout = old_stdout


class StdoutHandler(logging.StreamHandler):
    """a stream handler that writes to whatever ``sys.stdout`` is at the time of the record (tests and notebooks replace it)"""

    def __init__(self):
        super().__init__(sys.stdout)

    @property
    def stream(self):
        """the current ``sys.stdout``"""
        return sys.stdout

    @stream.setter
    def stream(self, _value):
        pass  # the base class constructor assigns it; the property above wins


class StreamDummy:
    """discards everything written to it"""

    def write(self, msg):
        """ignored"""

    def flush(self):
        """nothing to flush"""
