"""
Mixed-precision policy for model code that places its own casts.

The engine's ``torch_amp`` option uses torch's autocast, which decides per aten op and needs nothing from the model. This module
is the explicit alternative with the reference's API (returnn/frontend/amp.py): a process-wide policy naming the compute dtype;
``amp_cast_compute`` casts float tensors to it (for matmul-like ops), ``amp_cast_float32`` casts back (for normalisation,
exp / log, reductions and losses). Parameters stay float32 and are cast where they are used. Without a policy both are no-ops.
"""

from __future__ import annotations
from typing import Optional, Sequence, TypeVar, Union
from contextlib import contextmanager
from dataclasses import dataclass
from ..tensor import Tensor
from .dtype import is_float_dtype

__all__ = ["AmpPolicy", "get_amp_policy", "set_amp_policy", "set_amp_policy_ctx", "amp_cast_compute", "amp_cast_float32"]


@dataclass(frozen=True)
class AmpPolicy:
    """what mixed precision means for a run: the dtype of the matmul-like ops"""

    compute_dtype: str

    def __post_init__(self):
        if not is_float_dtype(self.compute_dtype):
            raise ValueError("AmpPolicy: compute_dtype %r is not a float dtype" % (self.compute_dtype,))


_policy: Optional[AmpPolicy] = None
T = TypeVar("T", bound=Optional[Tensor])


def get_amp_policy() -> Optional[AmpPolicy]:
    """the active policy, None outside mixed precision"""
    return _policy


def set_amp_policy(policy: Optional[Union[AmpPolicy, str]]):
    """``policy``: an :class:`AmpPolicy`, just the compute dtype (e.g. ``"bfloat16"``), or None to switch it off"""
    global _policy
    if isinstance(policy, str):
        policy = AmpPolicy(compute_dtype=policy)
    if policy is not None and not isinstance(policy, AmpPolicy):
        raise TypeError("set_amp_policy: expected AmpPolicy, str or None, got %r" % type(policy))
    _policy = policy


@contextmanager
def set_amp_policy_ctx(policy: Optional[Union[AmpPolicy, str]]):
    """policy for the duration of the block"""
    global _policy
    old = _policy
    try:
        set_amp_policy(policy)
        yield
    finally:
        _policy = old


def _to(x: Optional[Tensor], dtype: str) -> Optional[Tensor]:
    if x is None or x.dtype == dtype or not is_float_dtype(x.dtype):
        return x
    from .array_ import cast

    return cast(x, dtype)


def amp_cast_compute(*tensors: T) -> Union[T, Sequence[T]]:
    """float tensors -> the policy's compute dtype; None entries and other dtypes pass through; one tensor in, one tensor out"""
    res = tensors if _policy is None else tuple(_to(x, _policy.compute_dtype) for x in tensors)
    return res[0] if len(res) == 1 else res


def amp_cast_float32(*tensors: T) -> Union[T, Sequence[T]]:
    """float tensors -> float32 under a policy"""
    res = tensors if _policy is None else tuple(_to(x, "float32") for x in tensors)
    return res[0] if len(res) == 1 else res
