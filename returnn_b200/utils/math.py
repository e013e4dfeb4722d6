"""
Small numeric helpers: integer math, piecewise-linear and step functions of the training progress, number formatting,
seed mixing.

Parity: returnn/util/math.py (ceil_div :12, next_power_of_two :17, PiecewiseLinear :22, StepFunction :84,
simplify_and_format_number :152, merge_random_seeds :160).
"""

from __future__ import annotations
from typing import Dict, Sequence, Union
import bisect
import hashlib
import struct


def ceil_div(a: int, b: int) -> int:
    """ceil(a / b) in integers"""
    return -(-a // b)


def next_power_of_two(n: int) -> int:
    """smallest power of two >= n (1 for n <= 1)"""
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


class PiecewiseLinear:
    """linear interpolation between given points, constant outside; optional log-space interpolation"""

    def __init__(self, values: Dict[Union[int, float], Union[int, float]], *, kw_name: str = None, ignore_other_kwargs: bool = False):
        assert values
        self._xs = sorted(values.keys())
        self._ys = [values[x] for x in self._xs]
        self._kw_name = kw_name
        self._ignore_other_kwargs = ignore_other_kwargs

    def __call__(self, *args, **kwargs) -> float:
        if self._kw_name:
            x = kwargs.pop(self._kw_name)
            assert not args and (self._ignore_other_kwargs or not kwargs)
        else:
            (x,) = args
            assert not kwargs
        xs, ys = self._xs, self._ys
        if x <= xs[0]:
            return ys[0]
        if x >= xs[-1]:
            return ys[-1]
        i = bisect.bisect_right(xs, x)
        x0, x1, y0, y1 = xs[i - 1], xs[i], ys[i - 1], ys[i]
        return y0 + (y1 - y0) * (x - x0) / (x1 - x0)


class StepFunction:
    """piecewise constant: the value of the last point with key <= x (the first value before the first key)"""

    def __init__(self, values: Dict[Union[int, float], Union[int, float]], *, kw_name: str = None, ignore_other_kwargs: bool = False):
        assert values
        self._xs = sorted(values.keys())
        self._ys = [values[x] for x in self._xs]
        self._kw_name = kw_name
        self._ignore_other_kwargs = ignore_other_kwargs

    def __call__(self, *args, **kwargs):
        if self._kw_name:
            x = kwargs.pop(self._kw_name)
            assert not args and (self._ignore_other_kwargs or not kwargs)
        else:
            (x,) = args
            assert not kwargs
        i = bisect.bisect_right(self._xs, x)
        return self._ys[max(i - 1, 0)]


def simplify_and_format_number(n: Union[int, float]) -> str:
    """``3.0`` -> ``"3"``, other floats via repr"""
    if isinstance(n, float) and n.is_integer():
        return str(int(n))
    return str(n)


def merge_random_seeds(data_sources: Sequence[int], *, num_bytes: int = 4, signed: bool = False) -> int:
    """deterministic mix of several seeds into one integer of ``num_bytes`` bytes (order matters)"""
    h = hashlib.sha256()
    for s in data_sources:
        h.update(struct.pack("<q", int(s)))
    return int.from_bytes(h.digest()[:num_bytes], "little", signed=signed)
