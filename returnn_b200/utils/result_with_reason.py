"""
A result value together with an optional explanation.

Parity: returnn/util/result_with_reason.py (ResultWithReason :15).
"""

from __future__ import annotations
from dataclasses import dataclass
from typing import Generic, Optional, TypeVar

T = TypeVar("T")


@dataclass
class ResultWithReason(Generic[T]):
    """``result`` plus why"""

    result: T
    reason: Optional[str] = None

    def __bool__(self):
        return bool(self.result)
