"""
Loops: ``while_loop`` and ``scan`` run eagerly on the host; per-sequence ending is handled by masking the state update.

Parity: returnn/frontend/loop.py (while_loop, scan :82-222).
"""

from __future__ import annotations
from typing import Any, Callable, Optional, Sequence, Tuple, TypeVar, Union
import torch
from ..tensor import Tensor, Dim
from .tensor_array import TensorArray
from . import nested as _nested
from ._utils import wrap

__all__ = ["while_loop", "scan"]
S = TypeVar("S")
X = TypeVar("X")
Y = TypeVar("Y")


def while_loop(cond: Callable[[S], Union[bool, Tensor]], body: Callable[[S], S], initial: S) -> S:
    """``state = initial; while cond(state): state = body(state)``"""
    state = initial
    while True:
        c = cond(state)
        if isinstance(c, Tensor):
            assert not c.dims, "while_loop: cond must give a scalar"
            c = bool(c.raw_tensor)
        if not c:
            break
        state = body(state)
    return state


def scan(*, spatial_dim: Optional[Dim] = None, cond_dims: Optional[Sequence[Dim]] = None,
         cond_before_body: bool = True, initial: S = None, xs: X = None, ys: Y = None,
         cond: Optional[Callable[[X, S], Tensor]] = None, body: Callable[[X, S], Tuple[Y, S]],
         max_seq_len: Optional[Union[int, Tensor]] = None, return_tensor_arrays: bool = False) -> Tuple[Y, S, Dim]:
    """
    Iterate ``body(x_t, state) -> (y_t, state)`` over ``spatial_dim`` of ``xs`` (or until ``cond`` is False for all
    entries of ``cond_dims``).

    :param xs: nested structure of tensors having spatial_dim; sliced per step
    :param ys: nested structure of templates for the per-step outputs (structure only)
    :param cond: per-entry continuation condition over cond_dims; the out spatial dim gets per-entry sizes
    :return: stacked ys, final state, the spatial dim
    """
    if spatial_dim is not None and spatial_dim.is_dim_known() and cond is None:
        n = spatial_dim.get_dim_value()
        xs_arrays = _nested.tree_map(lambda x: TensorArray.unstack(x, axis=spatial_dim), xs)
        state = initial
        ys_arrays = None
        sizes = spatial_dim.get_size_tensor() if spatial_dim.is_dynamic() and spatial_dim.is_dynamic_seq_length() else None
        for i in range(n):
            x_t = _nested.tree_map(lambda a: a[i], xs_arrays) if xs is not None else None
            y_t, new_state = body(x_t, state)
            if sizes is not None and state is not None:
                # sequences that already ended keep their state
                from .array_ import where

                alive_raw = sizes.raw_tensor > i
                leaves = _nested.tree_flatten(new_state)
                dev = leaves[0].device if leaves and isinstance(leaves[0], Tensor) else None
                alive = wrap(alive_raw.to(dev) if dev else alive_raw, sizes.dims)

                def _sel(new, old):
                    if isinstance(new, Tensor) and all(d in new.dims for d in alive.dims):
                        return where(alive, new, old)
                    return new

                new_state = _nested.tree_map_multi(_sel, new_state, state)
            state = new_state
            if ys_arrays is None:
                ys_arrays = _nested.tree_map(lambda y: TensorArray(y.copy_template()), y_t)
            _nested.tree_map_multi(lambda arr, y: arr.push_back(y), ys_arrays, y_t)
        if ys_arrays is None:
            ys_arrays = _nested.tree_map(lambda y: TensorArray(y), ys)
        if return_tensor_arrays:
            return ys_arrays, state, spatial_dim
        out = _nested.tree_map(lambda arr: arr.stack(axis=spatial_dim), ys_arrays)
        return out, state, spatial_dim
    # dynamic ending via cond
    assert cond is not None and cond_dims is not None
    if spatial_dim is None:
        spatial_dim = Dim(None, name="scan-dim")
    state = initial
    ys_arrays = None
    i = 0
    max_len = int(max_seq_len.raw_tensor.max()) if isinstance(max_seq_len, Tensor) else max_seq_len
    ended = None
    lens = None
    x_t = None
    while True:
        if cond_before_body:
            c = cond(x_t, state)
        else:
            c = None
        if c is not None:
            alive = c.raw_tensor if ended is None else (c.raw_tensor & ~ended)
            if lens is None:
                lens = torch.zeros_like(alive, dtype=torch.int32)
            ended = ~alive if ended is None else (ended | ~alive)
            if not bool(alive.any()) or (max_len is not None and i >= max_len):
                break
            lens = lens + alive.to(torch.int32)
        y_t, state = body(x_t, state)
        if ys_arrays is None:
            ys_arrays = _nested.tree_map(lambda y: TensorArray(y.copy_template()), y_t)
        _nested.tree_map_multi(lambda arr, y: arr.push_back(y), ys_arrays, y_t)
        i += 1
        if not cond_before_body:
            c = cond(x_t, state)
            alive = c.raw_tensor if ended is None else (c.raw_tensor & ~ended)
            if lens is None:
                lens = torch.ones_like(alive, dtype=torch.int32)
            else:
                lens = lens + (~ended).to(torch.int32)
            ended = ~alive if ended is None else (ended | ~alive)
            if not bool(alive.any()) or (max_len is not None and i >= max_len):
                break
    if lens is not None:
        spatial_dim.dyn_size_ext = Tensor("%s:size" % spatial_dim.name, dims=list(cond_dims), dtype="int32", raw_tensor=lens.cpu())
    if ys_arrays is None:
        ys_arrays = _nested.tree_map(lambda y: TensorArray(y), ys)
    if return_tensor_arrays:
        return ys_arrays, state, spatial_dim
    return _nested.tree_map(lambda arr: arr.stack(axis=spatial_dim), ys_arrays), state, spatial_dim
