"""
Harness for RF model code: run a function of (model, batch) on a padded batch and again on every sequence of the batch alone, and
require equal results on the valid frames. A layer that lets padding leak into its output (an unmasked reduction, a convolution over
padded frames, a softmax over padded keys, statistics over padded frames) fails this, whatever its output values are.
The idea follows ``run_model`` of the reference's test helpers (tests/rf_utils.py:58-120); the implementation is this repository's.
"""

from __future__ import annotations
from typing import Callable, Dict, List, Optional, Sequence, Tuple
import torch

import returnn_b200.frontend as rf
from returnn_b200.tensor import Tensor, Dim, batch_dim


def make_batch(lens: Sequence[int], feat: Optional[Dim], *, seed: int = 0, dtype: str = "float32", sparse_dim: Optional[Dim] = None,
               time_name: str = "time") -> Tuple[Tensor, Dim]:
    """``[B, T(, F)]`` tensor with the given sequence lengths; padded frames hold LARGE values, so that a leak is visible"""
    g = torch.Generator().manual_seed(seed)
    B, T = len(lens), max(lens)
    batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(B, dtype=torch.int32))
    time = Dim(None, name=time_name)
    time.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor(list(lens), dtype=torch.int32))
    if sparse_dim is not None:
        raw = torch.randint(0, sparse_dim.dimension, (B, T), generator=g, dtype=torch.int64).to(torch.int32 if dtype == "int32" else torch.int64)
        for b, n in enumerate(lens):
            raw[b, n:] = sparse_dim.dimension - 1
        return Tensor("x", dims=[batch_dim, time], dtype=dtype, sparse_dim=sparse_dim, raw_tensor=raw), time
    raw = torch.randn(B, T, feat.dimension, generator=g)
    for b, n in enumerate(lens):
        raw[b, n:] = 1e3 * (1 + torch.rand(T - n, feat.dimension, generator=g))
    return Tensor("x", dims=[batch_dim, time, feat], dtype=dtype, feature_dim=feat, raw_tensor=raw), time


def single_seq(x: Tensor, time: Dim, b: int) -> Tuple[Tensor, Dim]:
    """sequence ``b`` of the batch as a batch of one, without padding"""
    n = int(time.dyn_size_ext.raw_tensor[b])
    t1 = Dim(None, name=time.name)
    t1.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([n], dtype=torch.int32))
    raw = x.raw_tensor[b: b + 1, :n].clone()
    dims = [batch_dim, t1] + list(x.dims[2:])
    return Tensor("x", dims=dims, dtype=x.dtype, sparse_dim=x.sparse_dim, feature_dim=x.feature_dim if x.feature_dim in dims else None, raw_tensor=raw), t1


def valid_rows(y: Tensor, out_time: Optional[Dim]) -> List[torch.Tensor]:
    """per sequence: ``[len_b, ...]`` if the output has a time axis, else the batch entry"""
    order = [batch_dim] + ([out_time] if out_time is not None and out_time in y.dims else [])
    rest = [d for d in y.dims if d not in order]
    raw = y.copy_transpose(order + rest).raw_tensor
    if len(order) == 1:
        return [raw[b] for b in range(raw.shape[0])]
    lens = out_time.dyn_size_ext.raw_tensor.tolist() if out_time.dyn_size_ext is not None and out_time.dyn_size_ext.dims else [raw.shape[1]] * raw.shape[0]
    return [raw[b, : int(n)] for b, n in enumerate(lens)]


def check_padding_invariance(fn: Callable[[Tensor, Dim], Tuple[Tensor, Optional[Dim]]], x: Tensor, time: Dim, *, atol: float = 1e-5,
                             rtol: float = 1e-4, train_flag: bool = False) -> List[torch.Tensor]:
    """
    :param fn: ``(x, time) -> (y, out_time or None)``; called once for the batch and once per sequence
    :return: the per-sequence results of the batched call
    """
    B = x.raw_tensor.shape[0]
    with torch.no_grad():
        rf.init_train_step_run_ctx(train_flag=train_flag, step=0, epoch=1)
        batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(B, dtype=torch.int32))
        y, out_time = fn(x, time)
        batched = [r.clone() for r in valid_rows(y, out_time)]
        for b in range(B):
            batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(1, dtype=torch.int32))
            xb, tb = single_seq(x, time, b)
            yb, otb = fn(xb, tb)
            alone = valid_rows(yb, otb)[0]
            assert alone.shape == batched[b].shape, "sequence %i: shape %s alone, %s in the batch" % (b, tuple(alone.shape), tuple(batched[b].shape))
            if alone.dtype.is_floating_point:
                assert torch.isfinite(alone).all(), "sequence %i alone is not finite" % b
                torch.testing.assert_close(batched[b], alone, atol=atol, rtol=rtol, msg=lambda m, b=b: "sequence %i: %s" % (b, m))
            else:
                assert torch.equal(batched[b], alone), "sequence %i differs" % b
    batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(B, dtype=torch.int32))
    return batched
