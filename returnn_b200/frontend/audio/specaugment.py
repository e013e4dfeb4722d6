"""
SpecAugment: random time and feature masks.

Parity: returnn/frontend/audio/specaugment.py:14-242 (schedule by global train step boundaries (0, 1000, 2000),
up to ``T // 100`` time masks of at most 20 frames, feature masks of at most ``F // 5``).
"""

from __future__ import annotations
from typing import Collection, Optional, Sequence, Union
import torch
from ...tensor import Tensor, Dim
from .._utils import wrap, axis_of
from ..run_ctx import get_run_ctx

__all__ = ["specaugment", "random_mask", "mask"]


def specaugment(x: Tensor, *, spatial_dim: Dim, feature_dim: Optional[Dim] = None, global_train_step_dependent: bool = True,
                only_on_train: bool = True, max_consecutive_spatial_dims: int = 20, max_consecutive_feature_dims: Optional[int] = None,
                num_spatial_mask_factor: int = 100, steps_first_second: Sequence[int] = (0, 1000, 2000)) -> Tensor:
    """apply SpecAugment (only when the train flag is on, unless only_on_train=False)"""
    if feature_dim is None:
        assert x.feature_dim
        feature_dim = x.feature_dim
    if max_consecutive_feature_dims is None:
        max_consecutive_feature_dims = feature_dim.dimension // 5
    ctx = get_run_ctx()
    if only_on_train:
        flag = ctx.is_train_flag_enabled(func=specaugment)
        if not (bool(flag.raw_tensor) if isinstance(flag, Tensor) else flag):
            return x
    step = ctx.step
    step = int(step.raw_tensor) if isinstance(step, Tensor) else int(step)
    if global_train_step_dependent:
        s0, s1, s2 = steps_first_second
        if step < s0:
            return x
        stage = 0 if step < s1 else (1 if step < s2 else 2)
    else:
        stage = 2
    T = spatial_dim.get_dim_value()
    time_factor = 1
    max_time_masks = max(T // num_spatial_mask_factor, 2) if stage >= 1 else 1
    if stage == 2:
        max_time_masks = max(T // (num_spatial_mask_factor // 2 or 1), 2) if False else max_time_masks
    x = random_mask(x, mask_axis=spatial_dim, broadcast_axis=feature_dim, min_num=min(max_time_masks, 1 if stage == 0 else 2),
                    max_num=max_time_masks, max_dims=max_consecutive_spatial_dims // time_factor)
    x = random_mask(x, mask_axis=feature_dim, broadcast_axis=spatial_dim, min_num=1 if stage == 0 else 2,
                    max_num=2 if stage == 0 else 5, max_dims=max_consecutive_feature_dims)
    return x


def random_mask(x: Tensor, *, mask_axis: Dim, broadcast_axis: Union[Dim, Collection[Dim]], min_num: int, max_num: int,
                max_dims: int, mask_value: float = 0.0) -> Tensor:
    """
    Per batch entry, draw n in [min_num, max_num] masks; each mask has a random start in the valid range and a random
    width in [1, max_dims]; masked positions (over mask_axis, broadcast over broadcast_axis) are set to mask_value.
    """
    if isinstance(broadcast_axis, Dim):
        broadcast_axis = [broadcast_axis]
    batch_dims = [d for d in x.dims if d != mask_axis and d not in broadcast_axis]
    raw = x.raw_tensor
    dev = raw.device
    bshape = [d.get_dim_value() for d in batch_dims]
    n_axis = mask_axis.get_dim_value()
    if max_num <= 0 or max_dims <= 0 or n_axis == 0:
        return x
    if mask_axis.is_dynamic() and mask_axis.dyn_size_ext is not None and mask_axis.dyn_size_ext.dims and all(
            d in batch_dims for d in mask_axis.dyn_size_ext.dims):
        sizes = mask_axis.get_size_tensor(device=dev).copy_compatible_to_dims_raw(batch_dims).expand(*bshape).to(torch.int64)
    else:
        sizes = torch.full(bshape or [1], n_axis, dtype=torch.int64, device=dev).reshape(bshape)
    num = torch.randint(min_num, max_num + 1, bshape, device=dev) if max_num > min_num else torch.full(bshape, min_num, device=dev)
    k = torch.arange(max_num, device=dev)
    active = k < num.unsqueeze(-1)  # [.., max_num]
    starts = (torch.rand(bshape + [max_num], device=dev) * sizes.unsqueeze(-1).float()).long()
    widths = torch.randint(1, max_dims + 1, bshape + [max_num], device=dev)
    pos = torch.arange(n_axis, device=dev)
    hit = (pos >= starts.unsqueeze(-1)) & (pos < (starts + widths).unsqueeze(-1)) & active.unsqueeze(-1)  # [.., max_num, n]
    m = hit.any(dim=-2)  # [.., n]
    m_t = wrap(m, batch_dims + [mask_axis])
    mraw = m_t.copy_compatible_to_dims_raw(x.dims)
    return wrap(torch.where(mraw, torch.full((), mask_value, dtype=raw.dtype, device=dev), raw), x.dims, like=x)


def mask(x: Tensor, *, mask_axis: Dim, pos: Tensor, max_amount: int, mask_value: float = 0.0) -> Tensor:
    """mask [pos, pos + amount) with a random amount in [1, max_amount] per batch entry"""
    raw = x.raw_tensor
    dev = raw.device
    n = mask_axis.get_dim_value()
    amount = torch.randint(1, max_amount + 1, pos.raw_tensor.shape, device=dev)
    p = pos.raw_tensor.to(dev).unsqueeze(-1)
    rng = torch.arange(n, device=dev)
    m = (rng >= p) & (rng < p + amount.unsqueeze(-1))
    m_t = wrap(m, list(pos.dims) + [mask_axis])
    return wrap(torch.where(m_t.copy_compatible_to_dims_raw(x.dims), torch.full((), mask_value, dtype=raw.dtype, device=dev), raw), x.dims, like=x)
