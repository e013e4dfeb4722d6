"""
Recording and replaying the draws of ``rf.random``: a journal keeps every drawn tensor (as a NumPy array) together with the
arguments of the call; replaying feeds the same arrays back in the same order. Two runs that must see identical random numbers
although their generators differ (the generic RF path against the fused executor, this framework against the reference, CPU against
GPU) record with one and replay with the other. The order of the calls must be the same in both runs; shapes and dtypes are checked.

    journal = RandomJournal()
    with journal.recording():
        y1 = model(x)          # draws are stored
    with journal.replaying():
        y2 = model_other(x)    # the same draws come back

Same role as returnn/frontend/_random_journal.py:19 (RandomJournal, RandomJournalEntry), without its graph-mode reader nodes.
"""

from __future__ import annotations
from typing import Any, List, Optional
from dataclasses import dataclass
import contextlib
import numpy

__all__ = ["RandomJournal", "RandomJournalEntry", "current_journal"]

_current: Optional["RandomJournal"] = None
_mode: Optional[str] = None  # "record" / "replay"


def current_journal():
    """(journal, mode) active in this thread of control, or (None, None)"""
    return _current, _mode


@dataclass
class RandomJournalEntry:
    """one draw"""

    out: numpy.ndarray
    dtype: str
    distribution: str
    mean: Any = None
    stddev: Any = None
    bound: Any = None
    minval: Any = None
    maxval: Any = None
    seed: Any = None
    static: Optional[bool] = None


class RandomJournal:
    """see the module docstring"""

    def __init__(self):
        self._entries: List[RandomJournalEntry] = []
        self._cur_entry_idx = 0

    def __len__(self):
        return len(self._entries)

    def append(self, *, out, dtype: str, distribution: str, **params):
        """store a draw (``out``: array-like)"""
        self._entries.append(RandomJournalEntry(out=numpy.array(out), dtype=dtype, distribution=distribution, **params))

    def get_next(self, *, shape=None, dtype: Optional[str] = None, distribution: Optional[str] = None) -> RandomJournalEntry:
        """the next stored draw; shape / dtype / distribution of the asking call are checked against it"""
        if self._cur_entry_idx >= len(self._entries):
            raise IndexError("random journal: draw %i asked for, %i recorded" % (self._cur_entry_idx + 1, len(self._entries)))
        entry = self._entries[self._cur_entry_idx]
        where = "random journal entry %i" % self._cur_entry_idx
        if shape is not None and tuple(shape) != tuple(entry.out.shape):
            raise ValueError("%s: recorded shape %s, asked for %s" % (where, tuple(entry.out.shape), tuple(shape)))
        if dtype is not None and dtype != entry.dtype:
            raise ValueError("%s: recorded dtype %s, asked for %s" % (where, entry.dtype, dtype))
        if distribution is not None and distribution != entry.distribution:
            raise ValueError("%s: recorded distribution %s, asked for %s" % (where, entry.distribution, distribution))
        self._cur_entry_idx += 1
        return entry

    def reached_end(self) -> bool:
        """all recorded draws were replayed"""
        return self._cur_entry_idx >= len(self._entries)

    def rewind(self):
        """replay from the first draw again"""
        self._cur_entry_idx = 0

    @contextlib.contextmanager
    def recording(self):
        """``rf.random`` stores its draws here inside the block"""
        global _current, _mode
        old = (_current, _mode)
        _current, _mode = self, "record"
        try:
            yield self
        finally:
            _current, _mode = old

    @contextlib.contextmanager
    def replaying(self):
        """``rf.random`` returns the stored draws inside the block"""
        global _current, _mode
        old = (_current, _mode)
        self.rewind()
        _current, _mode = self, "replay"
        try:
            yield self
        finally:
            _current, _mode = old
