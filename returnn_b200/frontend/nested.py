"""
Tree utilities over nested dict / list / tuple / State structures of tensors (own implementation, no extra dependency).
Parity: returnn/frontend/nested.py; the ``tree`` package use in the reference.
"""

from __future__ import annotations
from typing import Any, Callable, List, Sequence
from ..tensor import Tensor, Dim

__all__ = ["tree_flatten", "tree_map", "tree_map_multi", "tree_unflatten_like", "gather_nested", "masked_select_nested",
           "masked_scatter_nested", "mask_nested", "where_nested"]


def _is_leaf(x) -> bool:
    return not isinstance(x, (dict, list, tuple)) or isinstance(x, Tensor)


def tree_flatten(struct) -> List[Any]:
    """leaves in deterministic order (dict keys in insertion order); None leaves are skipped"""
    out = []

    def rec(x):
        if x is None:
            return
        if isinstance(x, dict):
            for v in x.values():
                rec(v)
        elif isinstance(x, (list, tuple)) and not isinstance(x, Tensor):
            for v in x:
                rec(v)
        else:
            out.append(x)

    rec(struct)
    return out


def tree_map(fn: Callable, struct):
    """same structure, fn applied to leaves"""
    if struct is None:
        return None
    if isinstance(struct, dict):
        res = struct.__class__.__new__(struct.__class__)
        dict.__init__(res)
        for k, v in struct.items():
            dict.__setitem__(res, k, tree_map(fn, v))
        return res
    if isinstance(struct, tuple) and hasattr(struct, "_fields"):
        return struct.__class__(*[tree_map(fn, v) for v in struct])
    if isinstance(struct, (list, tuple)):
        return struct.__class__(tree_map(fn, v) for v in struct)
    return fn(struct)


def tree_map_multi(fn: Callable, *structs):
    """fn(leaf_a, leaf_b, ...) over parallel structures"""
    first = structs[0]
    if first is None:
        return None
    if isinstance(first, dict):
        res = first.__class__.__new__(first.__class__)
        dict.__init__(res)
        for k in first:
            dict.__setitem__(res, k, tree_map_multi(fn, *[s[k] for s in structs]))
        return res
    if isinstance(first, tuple) and hasattr(first, "_fields"):
        return first.__class__(*[tree_map_multi(fn, *vs) for vs in zip(*structs)])
    if isinstance(first, (list, tuple)):
        return first.__class__(tree_map_multi(fn, *vs) for vs in zip(*structs))
    return fn(*structs)


def tree_unflatten_like(struct, leaves: Sequence[Any]):
    """inverse of tree_flatten"""
    it = iter(leaves)
    return tree_map(lambda _: next(it), struct)


def gather_nested(struct, *, indices: Tensor, dim_map=None):
    """rf.gather on every tensor that has the indexed dim (beam search: select states by back-references)"""
    from .array_ import gather

    axis = indices.sparse_dim

    def f(x):
        if isinstance(x, Tensor) and axis in x.dims:
            return gather(x, indices=indices, axis=axis)
        if isinstance(x, Dim) and dim_map and x in dim_map:
            return dim_map[x]
        return x

    return tree_map(f, struct)


def masked_select_nested(struct, *, mask: Tensor, dims, out_dim=None, dim_map=None):
    """rf.masked_select on every tensor having all mask dims"""
    from .array_ import masked_select

    state = {"out_dim": out_dim}

    def f(x):
        if isinstance(x, Tensor) and all(d in x.dims for d in dims):
            res, od = masked_select(x, mask=mask, dims=dims, out_dim=state["out_dim"])
            state["out_dim"] = od
            return res
        return x

    return tree_map(f, struct), state["out_dim"]


def masked_scatter_nested(struct, backup, *, mask: Tensor, dims, in_dim, dim_map=None):
    """rf.masked_scatter on every tensor having in_dim"""
    from .array_ import masked_scatter

    def f(x, b):
        if isinstance(x, Tensor) and in_dim in x.dims:
            return masked_scatter(x, b, mask=mask, dims=dims, in_dim=in_dim)
        return x

    return tree_map_multi(f, struct, backup)


def where_nested(cond: Tensor, a, b):
    """rf.where over parallel structures"""
    from .array_ import where

    def f(x, y):
        if isinstance(x, Tensor):
            return where(cond, x, y)
        return x

    return tree_map_multi(f, a, b)


def mask_nested(struct, *, mask: Tensor, mask_value):
    """where(mask, x, mask_value[x]) over the structure"""
    return where_nested(mask, struct, mask_value)
