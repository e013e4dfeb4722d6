"""Iterator with a put-back queue (the engine splits a batch that does not fit and pushes the halves back). Parity: returnn/torch/data/queued_data_iter.py."""

from __future__ import annotations
from typing import Iterable, Iterator, List, Sequence, TypeVar, Union

T = TypeVar("T")


class QueuedDataIter:
    """wraps an iterator; items given to :meth:`extend` come out first, in their order"""

    def __init__(self, original_iter: Union[Iterable[T], Iterator[T]]):
        self._iter = iter(original_iter)
        self._front: List[T] = []

    def extend(self, items: Sequence[T]):
        """the next items of ``__next__`` will be these, in the same order, before the wrapped iterator continues"""
        self._front[0:0] = list(items)

    def __iter__(self):
        return self

    def __next__(self) -> T:
        if self._front:
            return self._front.pop(0)
        return next(self._iter)
