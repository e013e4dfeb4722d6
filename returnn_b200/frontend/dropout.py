"""
Dropout.  Parity: returnn/frontend/dropout.py:69-101 (noise shape by ``axis``, scale 1/keep, train-flag gating;
``rf_dropout_broadcast`` config default).
"""

from __future__ import annotations
from typing import Optional, Sequence, Union
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap
from .run_ctx import get_run_ctx

__all__ = ["dropout", "dropout_broadcast_default"]


def dropout(source: Tensor, drop_prob: Union[float, Tensor], *, axis: Optional[Union[Dim, Sequence[Dim], bool]] = None,
            on_forward: bool = False) -> Tensor:
    """
    :param drop_prob: probability of zeroing
    :param axis: the noise is drawn only over these dims and broadcast over the others.
        None/True with broadcasting enabled: over batch+spatial dims sharing one mask per... all dims (no broadcast).
    :param on_forward: also apply outside of training
    """
    if isinstance(drop_prob, (int, float)) and not drop_prob:
        return source
    train = get_run_ctx().is_train_flag_enabled(func=dropout)
    if not on_forward and not (bool(train._raw_tensor) if isinstance(train, Tensor) else train):
        return source
    p = float(drop_prob._raw_tensor) if isinstance(drop_prob, Tensor) else float(drop_prob)
    keep = 1.0 - p
    raw = source._raw_tensor
    if axis is None or axis is True or axis is False:
        if raw.is_cuda and raw.dtype == torch.bfloat16:
            from ..ops import elementwise as _ew

            if _ew.available():
                return wrap(_ew.dropout(raw, p), source._dims, like=source)
        return wrap(torch.nn.functional.dropout(raw, p, training=True), source._dims, like=source)
    axes = [axis] if isinstance(axis, Dim) else list(axis)
    shape = [raw.shape[i] if d in axes else 1 for i, d in enumerate(source._dims)]
    mask = torch.empty(shape, dtype=raw.dtype, device=raw.device).bernoulli_(keep)
    return wrap(raw * mask * (1.0 / keep), source._dims, like=source)


def dropout_broadcast_default() -> bool:
    """config ``rf_dropout_broadcast``; True up to behavior version 18, then False"""
    from ..config import get_global_config
    from ..utils.basic import BehaviorVersion

    cfg = get_global_config(raise_exception=False)
    if cfg and cfg.has("rf_dropout_broadcast"):
        return cfg.bool("rf_dropout_broadcast", True)
    return BehaviorVersion.get() <= 18
