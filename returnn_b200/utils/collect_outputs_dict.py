"""
A dict that keeps only keys matching given wildcard patterns (to collect selected intermediate outputs of a model).

Parity: returnn/util/collect_outputs_dict.py (CollectOutputsDict :12, is_key_allowed_in_collect_outputs_dict :69).
"""

from __future__ import annotations
from typing import Optional, Sequence, Union
import fnmatch


class CollectOutputsDict(dict):
    """assignments of keys that match no pattern are dropped silently"""

    def __init__(self, *args, allowed_key_patterns: Optional[Sequence[str]] = None, **kwargs):
        self.allowed_key_patterns = list(allowed_key_patterns) if allowed_key_patterns is not None else None
        super().__init__()
        self.update(dict(*args, **kwargs))

    def is_key_allowed(self, key: str) -> bool:
        """:return: no patterns given, or ``key`` matches one"""
        pats = self.allowed_key_patterns
        return pats is None or any(fnmatch.fnmatchcase(key, p) for p in pats)

    def __setitem__(self, key, value):
        if self.is_key_allowed(key):
            dict.__setitem__(self, key, value)

    def setdefault(self, key, default=None):
        if not self.is_key_allowed(key):
            return None
        return dict.setdefault(self, key, default)

    def update(self, mapping=(), **kwargs):
        items = mapping.items() if hasattr(mapping, "items") else mapping
        for k, v in list(items) + list(kwargs.items()):
            self[k] = v


def is_key_allowed_in_collect_outputs_dict(collect_outputs: Union[CollectOutputsDict, dict], key: str) -> bool:
    """plain dicts take every key"""
    return collect_outputs.is_key_allowed(key) if isinstance(collect_outputs, CollectOutputsDict) else True
