"""
Reductions over named dims, with masking of padded frames, plus ``top_k`` and ``RunningMean``.

Parity: returnn/frontend/reduce.py:1-314 (top_k :278); masking semantics
returnn/torch/frontend/_backend.py:1813-1873.
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap, axis_of, torch_dtype
from .module import Module
from .parameter import Parameter

__all__ = ["reduce", "reduce_sum", "reduce_max", "reduce_min", "reduce_mean", "reduce_logsumexp", "reduce_logmeanexp",
           "reduce_any", "reduce_all", "reduce_argmin", "reduce_argmax", "reduce_out", "RunningMean", "top_k"]


def _neutral(mode: str, dtype: torch.dtype):
    if mode in ("sum", "mean", "any"):
        return 0
    if mode == "all":
        return 1
    if mode in ("max", "argmax", "logsumexp", "logmeanexp"):
        return float("-inf") if dtype.is_floating_point else torch.iinfo(dtype).min
    if mode in ("min", "argmin"):
        return float("inf") if dtype.is_floating_point else torch.iinfo(dtype).max
    raise ValueError(mode)


def reduce(source: Tensor, *, mode: str, axis: Union[Dim, Sequence[Dim]], use_mask: bool = True, distributed: bool = False) -> Tensor:
    """
    :param mode: sum, max, min, mean, logsumexp, logmeanexp, any, all, argmin, argmax
    :param axis: dim(s) to reduce
    :param use_mask: ignore padded frames of dynamic axes
    :param distributed: additionally reduce over all ranks (sum/max/min/mean)
    """
    from . import _numpy_backend as _np

    if _np.is_numpy(source):
        return _np.NumpyBackend.reduce(source, mode=mode, axis=axis, use_mask=use_mask)
    axes = [axis] if isinstance(axis, Dim) else list(axis)
    raw = source._raw_tensor
    idxs = [axis_of(source, d) for d in axes]
    n_mask_elems = None
    if use_mask:
        for d in axes:
            if d.is_dynamic() and not d.is_batch_dim() and d.need_masking() and d.dyn_size_ext is not None and d.dyn_size_ext.dims:
                mask = d.get_mask(device=raw.device)
                mraw = mask.copy_compatible_to_dims_raw(source._dims)
                raw = torch.where(mraw, raw, torch.full((), _neutral(mode, raw.dtype), dtype=raw.dtype, device=raw.device))
                if mode in ("mean", "logmeanexp"):
                    cnt = d.get_size_tensor(device=raw.device)
                    n_mask_elems = (cnt, d) if n_mask_elems is None else n_mask_elems
    if mode in ("argmax", "argmin"):
        assert len(idxs) == 1
        out = (torch.argmax if mode == "argmax" else torch.argmin)(raw, dim=idxs[0]).to(torch.int32)
        dims = [d for i, d in enumerate(source._dims) if i != idxs[0]]
        return wrap(out, dims, sparse_dim=axes[0])
    if mode == "sum":
        out = torch.sum(raw, dim=idxs)
    elif mode == "max":
        out = torch.amax(raw, dim=idxs)
    elif mode == "min":
        out = torch.amin(raw, dim=idxs)
    elif mode == "mean":
        if n_mask_elems is None:
            out = torch.mean(raw, dim=idxs)
        else:
            # number of valid elements over the reduced axes, per remaining index
            from .array_ import num_elements_of_shape

            tot = torch.sum(raw, dim=idxs)
            cnt, dyn_d = n_mask_elems
            remaining = [d for i, d in enumerate(source._dims) if i not in idxs]
            other = 1
            for d in axes:
                if d != dyn_d and d not in cnt._dims:
                    other *= d.get_dim_value()
            if all(dd in axes for dd in cnt._dims):
                denom = float(int(cnt._raw_tensor.sum()) * other)
                out = tot / denom
            else:
                craw = cnt.copy_compatible_to_dims_raw(remaining).to(tot.dtype) * other
                out = tot / craw
    elif mode in ("logsumexp", "logmeanexp"):
        out = torch.logsumexp(raw, dim=idxs)
        if mode == "logmeanexp":
            import math

            if n_mask_elems is None:
                n = 1
                for i in idxs:
                    n *= raw.shape[i]
                out = out - math.log(n)
            else:
                cnt, dyn_d = n_mask_elems
                remaining = [d for i, d in enumerate(source._dims) if i not in idxs]
                out = out - torch.log(cnt.copy_compatible_to_dims_raw(remaining).to(out.dtype))
    elif mode == "any":
        out = raw
        for i in sorted(idxs, reverse=True):
            out = torch.any(out, dim=i)
    elif mode == "all":
        out = raw
        for i in sorted(idxs, reverse=True):
            out = torch.all(out, dim=i)
    else:
        raise ValueError("reduce: invalid mode %r" % mode)
    dims = [d for i, d in enumerate(source._dims) if i not in idxs]
    res = wrap(out, dims, like=source)
    if distributed:
        from ..torch.util.distributed import all_reduce_differentiable

        op = {"sum": "sum", "mean": "avg", "max": "max", "min": "min"}[mode]
        res = wrap(all_reduce_differentiable(res._raw_tensor, op), dims, like=source)
    return res


def reduce_sum(source, *, axis, use_mask=True, distributed=False):
    """sum"""
    return reduce(source, mode="sum", axis=axis, use_mask=use_mask, distributed=distributed)


def reduce_max(source, *, axis, use_mask=True, distributed=False):
    """max"""
    return reduce(source, mode="max", axis=axis, use_mask=use_mask, distributed=distributed)


def reduce_min(source, *, axis, use_mask=True, distributed=False):
    """min"""
    return reduce(source, mode="min", axis=axis, use_mask=use_mask, distributed=distributed)


def reduce_mean(source, *, axis, use_mask=True, distributed=False):
    """mean"""
    return reduce(source, mode="mean", axis=axis, use_mask=use_mask, distributed=distributed)


def reduce_logsumexp(source, *, axis, use_mask=True):
    """log sum exp"""
    return reduce(source, mode="logsumexp", axis=axis, use_mask=use_mask)


def reduce_logmeanexp(source, *, axis, use_mask=True):
    """log mean exp"""
    return reduce(source, mode="logmeanexp", axis=axis, use_mask=use_mask)


def reduce_any(source, *, axis, use_mask=True):
    """logical or"""
    return reduce(source, mode="any", axis=axis, use_mask=use_mask)


def reduce_all(source, *, axis, use_mask=True):
    """logical and"""
    return reduce(source, mode="all", axis=axis, use_mask=use_mask)


def reduce_argmin(source, *, axis, use_mask=True):
    """argmin"""
    return reduce(source, mode="argmin", axis=axis, use_mask=use_mask)


def reduce_argmax(source, *, axis, use_mask=True):
    """argmax"""
    return reduce(source, mode="argmax", axis=axis, use_mask=use_mask)


def reduce_out(source: Tensor, *, mode: str, num_pieces: int, out_dim: Optional[Dim] = None) -> Tensor:
    """maxout-style: split the feature dim into (out_dim, num_pieces) and reduce over the pieces"""
    from .array_ import split_dims

    fd = source.feature_dim
    assert fd is not None and fd.dimension % num_pieces == 0
    if out_dim is None:
        out_dim = fd // num_pieces
    pieces = Dim(num_pieces, name="pieces")
    x = split_dims(source, axis=fd, dims=[out_dim, pieces])
    res = reduce(x, mode=mode, axis=pieces)
    res._feature_dim = out_dim
    return res


class RunningMean(Module):
    """exponential running mean over update steps; in eval the stored mean is returned"""

    def __init__(self, in_dim: Union[Dim, Sequence[Dim]], *, alpha: float, dtype: Optional[str] = None,
                 is_prob_distribution: Optional[bool] = None, update_only_in_train: bool = True):
        super().__init__()
        self.in_dim = in_dim
        self.shape = (in_dim,) if isinstance(in_dim, Dim) else tuple(in_dim)
        self.alpha = alpha
        self.is_prob_distribution = is_prob_distribution
        self.update_only_in_train = update_only_in_train
        self.mean = Parameter(self.shape, dtype=dtype, auxiliary=True)
        if is_prob_distribution:
            assert in_dim.dimension is not None
            self.mean.initial = 1.0 / in_dim.dimension

    def __call__(self, x: Tensor) -> Tensor:
        from .run_ctx import get_run_ctx

        def _update():
            x_ = reduce_mean(x, axis=[d for d in x.dims if d not in self.shape])
            new = self.mean + self.alpha * (x_ - self.mean)
            self.mean.assign(new)
            return new

        if not self.update_only_in_train or get_run_ctx().is_train_flag_enabled(func=RunningMean.__call__):
            with torch.no_grad():
                _update()
        return self.mean


def top_k(source: Tensor, *, axis: Union[Dim, Sequence[Dim]], k: Optional[Union[int, Tensor]] = None,
          k_dim: Optional[Dim] = None, sorted: bool = True) -> Tuple[Tensor, Union[Tensor, Sequence[Tensor]], Dim]:
    """
    k largest entries along axis (or jointly over several axes, as in beam search over ``[beam, vocab]``).

    :return: values [.., k_dim], indices (one per axis; sparse over that axis), k_dim
    """
    if k is None:
        assert k_dim is not None
        k = k_dim.get_dim_value()
    kk = int(k._raw_tensor) if isinstance(k, Tensor) else int(k)
    if k_dim is None:
        k_dim = Dim(kk, name="top-k")
    if isinstance(axis, (list, tuple)):
        axes = list(axis)
        rest = [d for d in source._dims if d not in axes]
        raw = source.copy_compatible_to_dims_raw(rest + axes)
        sizes = [raw.shape[len(rest) + i] for i in range(len(axes))]
        flat = raw.reshape(list(raw.shape[: len(rest)]) + [-1])
        kk_ = min(kk, flat.shape[-1])
        vals, idx = torch.topk(flat, kk_, dim=-1, sorted=sorted)
        if kk_ < kk:
            padn = kk - kk_
            vals = torch.nn.functional.pad(vals, [0, padn], value=float("-inf"))
            idx = torch.nn.functional.pad(idx, [0, padn], value=0)
        indices = []
        rem = idx
        for s, d in zip(reversed(sizes), reversed(axes)):
            indices.insert(0, wrap((rem % s).to(torch.int32), rest + [k_dim], sparse_dim=d))
            rem = torch.div(rem, s, rounding_mode="floor")
        return wrap(vals, rest + [k_dim], like=source), indices, k_dim
    ax = axis_of(source, axis)
    raw = source._raw_tensor
    if axis.is_dynamic() and axis.need_masking() and axis.is_dynamic_seq_length():
        m = axis.get_mask(device=raw.device).copy_compatible_to_dims_raw(source._dims)
        raw = torch.where(m, raw, torch.full((), _neutral("max", raw.dtype), dtype=raw.dtype, device=raw.device))
    vals, idx = torch.topk(raw, kk, dim=ax, sorted=sorted)
    dims = list(source._dims)
    dims[ax] = k_dim
    return wrap(vals, dims, like=source), wrap(idx.to(torch.int32), dims, sparse_dim=axis), k_dim
