"""
``matmul`` with named dims: contract over ``reduce``; dims common to both operands are batch dims; the rest are kept.

Parity: returnn/frontend/matmul.py; returnn/torch/frontend/_backend.py:1677-1787.
"""

from __future__ import annotations
from typing import Sequence, Union
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap

__all__ = ["matmul", "dot"]


def matmul(a: Tensor, b: Tensor, *, reduce: Union[Dim, Sequence[Dim]], use_mask: bool = True) -> Tensor:
    """
    :param reduce: dim(s) summed over; must be in both a and b
    :param use_mask: zero the padded frames of dynamic reduce dims first
    :return: dims = common (batch) dims, a-only dims, b-only dims
    """
    red = [reduce] if isinstance(reduce, Dim) else list(reduce)
    if use_mask:
        for d in red:
            if d.is_dynamic() and not d.is_batch_dim() and d.need_masking() and d.dyn_size_ext is not None and d.dyn_size_ext.dims:
                a = a.copy_masked(0, dims=[d])
    ad, bd = a._dims, b._dims
    a_raw, b_raw = a._raw_tensor, b._raw_tensor
    if a_raw.dtype != b_raw.dtype:
        if torch.is_autocast_enabled() and a_raw.is_floating_point():
            pass
        else:
            common_dtype = torch.promote_types(a_raw.dtype, b_raw.dtype)
            a_raw, b_raw = a_raw.to(common_dtype), b_raw.to(common_dtype)
    # fast path: x[..., in] @ w[in, out]
    if len(red) == 1 and len(bd) == 2 and ad and ad[-1] == red[0] and bd[0] == red[0] and bd[1] not in ad:
        if a_raw.is_cuda:
            # the same route as rf.Linear: the tcgen05 GEMM with its own backward (bf16 operands, i.e. bf16 tensors or autocast),
            # torch.matmul where that does not apply (fp32 without autocast, pitches that are not multiples of 8)
            from ..ops import linear as _linear

            out = _linear.linear(a_raw, b_raw)
        else:
            out = torch.matmul(a_raw, b_raw)
        res = wrap(out, tuple(ad[:-1]) + (bd[1],), feature_dim=bd[1])
        return res
    common = [d for d in ad if d in bd and d not in red]
    a_only = [d for d in ad if d not in bd]
    b_only = [d for d in bd if d not in ad]
    for d in red:
        assert d in ad and d in bd, "matmul: reduce dim %r must be in both %r and %r" % (d, a, b)
    a2 = a.copy_with_raw(a_raw).copy_compatible_to_dims_raw(common + a_only + red)
    b2 = b.copy_with_raw(b_raw).copy_compatible_to_dims_raw(common + red + b_only)
    cshape = list(a2.shape[: len(common)])
    ao_shape = list(a2.shape[len(common): len(common) + len(a_only)])
    r_shape = list(a2.shape[len(common) + len(a_only):])
    bo_shape = list(b2.shape[len(common) + len(red):])

    def _prod(xs):
        p = 1
        for x in xs:
            p *= x
        return p

    a3 = a2.reshape(cshape + [_prod(ao_shape), _prod(r_shape)])
    b3 = b2.reshape(cshape + [_prod(r_shape), _prod(bo_shape)])
    if a3.is_cuda and cshape:
        # batched products on the own GEMM where its shape rules hold (ops/bmm.py), torch.matmul otherwise
        from ..ops import bmm as _bmm

        bt = _prod(cshape)
        out = _bmm.bmm(a3.reshape(bt, a3.shape[-2], a3.shape[-1]), b3.reshape(bt, b3.shape[-2], b3.shape[-1])).reshape(cshape + ao_shape + bo_shape)
    else:
        out = torch.matmul(a3, b3).reshape(cshape + ao_shape + bo_shape)
    out_dims = common + a_only + b_only
    fd = None
    if b_only and b.feature_dim in b_only:
        fd = b.feature_dim
    elif a_only and a.feature_dim in a_only:
        fd = a.feature_dim
    return wrap(out, out_dims, feature_dim=fd)


dot = matmul  # the general contraction under its other name (reference: returnn/frontend/matmul.py:47)
