"""
Normalization layers.

Parity: returnn/frontend/normalization.py:25-440 (moments :25-85, LayerNorm :88, RMSNorm, GroupNorm, BatchNorm :267-365
with eps 1e-3 / momentum 0.1 / masked statistics, Normalize).
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union
import torch
from ..tensor import Tensor, Dim
from .module import Module
from .parameter import Parameter
from ._utils import wrap, axis_of
from .reduce import reduce_sum as _reduce_sum, reduce_mean as _reduce_mean
from . import math_ as _m
from .run_ctx import get_run_ctx

__all__ = ["moments", "LayerNorm", "RMSNorm", "GroupNorm", "GroupNormSpatial", "BatchNorm", "normalize", "Normalize",
           "batch_norm_distributed_default"]


def moments(x: Tensor, axis: Union[Dim, Sequence[Dim]], *, use_mask: bool = True, correction: Union[int, float] = 0,
            distributed: bool = False) -> Tuple[Tensor, Tensor]:
    """
    mean and variance over axis (padded frames excluded).

    :param distributed: statistics over all ranks: sums and counts are all-reduced (differentiably)
    """
    axes = [axis] if isinstance(axis, Dim) else list(axis)
    if distributed:
        from .array_ import num_elements_of_shape
        from ..torch.util.distributed import all_reduce_differentiable

        x32 = x if x.dtype in ("float32", "float64") else wrap(x._raw_tensor.float(), x._dims)
        s = _reduce_sum(x32, axis=axes, use_mask=use_mask)
        sq = _reduce_sum(x32 * x32, axis=axes, use_mask=use_mask)
        n = float(num_elements_of_shape(axes, use_mask=use_mask))
        packed = torch.cat([s._raw_tensor.reshape(-1), sq._raw_tensor.reshape(-1), torch.tensor([n], device=s._raw_tensor.device, dtype=s._raw_tensor.dtype)])
        packed = all_reduce_differentiable(packed, "sum")
        k = s._raw_tensor.numel()
        n_tot = packed[-1]
        mean_raw = (packed[:k] / n_tot).reshape(s._raw_tensor.shape)
        var_raw = (packed[k: 2 * k] / n_tot).reshape(s._raw_tensor.shape) - mean_raw * mean_raw
        if correction:
            var_raw = var_raw * (n_tot / (n_tot - correction))
        return wrap(mean_raw.to(x._raw_tensor.dtype), s._dims), wrap(var_raw.clamp_min(0).to(x._raw_tensor.dtype), s._dims)
    mean = _reduce_mean(x, axis=axes, use_mask=use_mask)
    diff = x - mean
    if correction:
        from .array_ import num_elements_of_shape

        n = num_elements_of_shape(axes, use_mask=use_mask)
        var = _reduce_sum(diff * diff, axis=axes, use_mask=use_mask) / (n - correction)
    else:
        var = _reduce_mean(diff * diff, axis=axes, use_mask=use_mask)
    return mean, var


class LayerNorm(Module):
    """layer norm over in_dim (one or several dims), eps 1e-6"""

    def __init__(self, in_dim: Union[Dim, Sequence[Dim]], *, eps: float = 1e-6, with_bias: bool = True):
        super().__init__()
        self.in_dim = in_dim
        self.eps = eps
        self.scale = Parameter([in_dim] if isinstance(in_dim, Dim) else list(in_dim))
        self.scale.initial = 1.0
        self.bias = None
        if with_bias:
            self.bias = Parameter(self.scale.dims)
            self.bias.initial = 0.0

    def __call__(self, x: Tensor) -> Tensor:
        if isinstance(self.in_dim, Dim) and x._dims and x._dims[-1] == self.in_dim:
            from ..ops import layer_norm as _ln

            out = _ln.layer_norm(x._raw_tensor, self.scale._raw_tensor, self.bias._raw_tensor if self.bias is not None else None, self.eps)
            return wrap(out, x._dims, like=x)
        mean, var = moments(x, self.in_dim)
        norm = (x - mean) * _m.rsqrt(var + self.eps)
        out = norm * self.scale
        return out + self.bias if self.bias is not None else out


class RMSNorm(Module):
    """x / sqrt(mean(x^2) + eps) * scale"""

    def __init__(self, in_dim: Union[Dim, Sequence[Dim]], *, eps: float = 1e-6, with_bias: bool = False):
        super().__init__()
        self.in_dim = in_dim
        self.eps = eps
        self.scale = Parameter([in_dim] if isinstance(in_dim, Dim) else list(in_dim))
        self.scale.initial = 1.0
        self.bias = None
        if with_bias:
            self.bias = Parameter(self.scale.dims)
            self.bias.initial = 0.0

    def __call__(self, x: Tensor) -> Tensor:
        if isinstance(self.in_dim, Dim) and x._dims and x._dims[-1] == self.in_dim:
            from ..ops import layer_norm as _ln

            out = _ln.rms_norm(x._raw_tensor, self.scale._raw_tensor, self.bias._raw_tensor if self.bias is not None else None, self.eps)
            return wrap(out, x._dims, like=x)
        var = _reduce_mean(_m.square(x), axis=self.in_dim)
        out = x * _m.rsqrt(var + self.eps) * self.scale
        return out + self.bias if self.bias is not None else out


class GroupNorm(Module):
    """group norm: statistics per group over (group features) — per frame, no pooling over time"""

    def __init__(self, in_dim: Dim, *, num_groups: Union[int, Dim], eps: float = 1e-6, with_bias: bool = True):
        super().__init__()
        self.in_dim = in_dim
        self.num_groups = num_groups if isinstance(num_groups, Dim) else Dim(num_groups, name="groups")
        self.eps = eps
        self.scale = Parameter([in_dim])
        self.scale.initial = 1.0
        self.bias = None
        if with_bias:
            self.bias = Parameter([in_dim])
            self.bias.initial = 0.0

    def __call__(self, x: Tensor) -> Tensor:
        from .array_ import split_dims, merge_dims

        per = self.in_dim.div_left(self.num_groups)
        xg = split_dims(x, axis=self.in_dim, dims=[self.num_groups, per])
        mean, var = moments(xg, per)
        xg = (xg - mean) * _m.rsqrt(var + self.eps)
        out, _ = merge_dims(xg, dims=[self.num_groups, per], out_dim=self.in_dim)
        out = out * self.scale
        return out + self.bias if self.bias is not None else out


class GroupNormSpatial(GroupNorm):
    """group norm with statistics pooled over the spatial dim too (the usual vision GroupNorm), masked"""

    def __call__(self, x: Tensor, *, spatial_dim: Dim) -> Tensor:
        from .array_ import split_dims, merge_dims

        per = self.in_dim.div_left(self.num_groups)
        xg = split_dims(x, axis=self.in_dim, dims=[self.num_groups, per])
        mean, var = moments(xg, [per, spatial_dim])
        xg = (xg - mean) * _m.rsqrt(var + self.eps)
        out, _ = merge_dims(xg, dims=[self.num_groups, per], out_dim=self.in_dim)
        out = out * self.scale
        return out + self.bias if self.bias is not None else out


class BatchNorm(Module):
    """
    Batch norm over all dims except in_dim. ``use_mask``: padded frames are excluded from the statistics.
    Running statistics are auxiliary parameters (buffers in the checkpoint).
    """

    def __init__(self, in_dim: Dim, *, affine: bool = True, momentum: float = 0.1, eps: float = 1e-3,
                 track_running_stats: bool = True, use_mask: Optional[bool] = None):
        super().__init__()
        assert isinstance(in_dim, Dim)
        self.in_dim = in_dim
        self.use_mask = use_mask
        self.momentum = momentum
        self.eps = eps
        self.running_mean = None
        self.running_variance = None
        if track_running_stats:
            self.running_mean = Parameter([in_dim], auxiliary=True)
            self.running_mean.initial = 0.0
            self.running_variance = Parameter([in_dim], auxiliary=True)
            self.running_variance.initial = 1.0
        self.affine = affine
        self.gamma = None
        self.beta = None
        if affine:
            self.gamma = Parameter([in_dim])
            self.gamma.initial = 1.0
            self.beta = Parameter([in_dim])
            self.beta.initial = 0.0

    def __call__(self, source: Tensor) -> Tensor:
        assert self.in_dim in source._dims
        train_flag = get_run_ctx().is_train_flag_enabled(func=BatchNorm.__call__)
        train = bool(train_flag._raw_tensor) if isinstance(train_flag, Tensor) else bool(train_flag)
        use_mask = self.use_mask
        if use_mask is None:
            from ..config import get_global_config

            cfg = get_global_config(raise_exception=False)
            use_mask = cfg.bool("rf_batch_norm_use_mask", False) if cfg else False
        distributed = False
        cfg = None
        try:
            from ..config import get_global_config

            cfg = get_global_config(raise_exception=False)
        except Exception:
            pass
        if cfg and cfg.bool("rf_batch_norm_distributed", False):
            distributed = True
        any_dyn = any(d.is_dynamic() and d.need_masking() and d.is_dynamic_seq_length() for d in source._dims)
        if not (use_mask and any_dyn) and not distributed:
            ax = axis_of(source, self.in_dim)
            raw = source._raw_tensor.movedim(ax, 1) if ax != 1 else source._raw_tensor
            if raw.ndim == 2:
                raw = raw.unsqueeze(-1)
            out = torch.nn.functional.batch_norm(
                raw, self.running_mean._raw_tensor if self.running_mean is not None else None,
                self.running_variance._raw_tensor if self.running_variance is not None else None,
                self.gamma._raw_tensor if self.affine else None, self.beta._raw_tensor if self.affine else None,
                training=train or self.running_mean is None, momentum=self.momentum, eps=self.eps)
            if source._raw_tensor.ndim == 2:
                out = out.squeeze(-1)
            if ax != 1:
                out = out.movedim(1, ax)
            return wrap(out, source._dims, like=source)
        if train or self.running_mean is None:
            mean, var = moments(source, [d for d in source._dims if d != self.in_dim], use_mask=use_mask, distributed=distributed)
            if self.running_mean is not None:
                with torch.no_grad():
                    self.running_mean._raw_tensor.lerp_(mean._raw_tensor.detach().to(self.running_mean._raw_tensor.dtype), self.momentum)
                    self.running_variance._raw_tensor.lerp_(var._raw_tensor.detach().to(self.running_variance._raw_tensor.dtype), self.momentum)
        else:
            mean, var = self.running_mean, self.running_variance
        out = (source - mean) * _m.rsqrt(var + self.eps)
        if self.affine:
            out = out * self.gamma + self.beta
        return out


def normalize(a: Tensor, *, axis: Union[Dim, Sequence[Dim]], epsilon: float = 1e-6) -> Tensor:
    """(a - mean) / sqrt(var + eps) over axis"""
    mean, var = moments(a, axis)
    return (a - mean) * _m.rsqrt(var + epsilon)


class Normalize(Module):
    """:func:`normalize` with optional learned scale and bias over param_dims"""

    def __init__(self, *, param_dims: Union[Dim, Sequence[Dim]], epsilon: float = 1e-6, scale: bool = True, bias: bool = True):
        super().__init__()
        self.epsilon = epsilon
        if isinstance(param_dims, Dim):
            param_dims = [param_dims]
        self.scale = None
        if scale:
            self.scale = Parameter(dims=param_dims)
            self.scale.initial = 1.0
        self.bias = None
        if bias:
            self.bias = Parameter(dims=param_dims)
            self.bias.initial = 0.0

    def __call__(self, a: Tensor, *, axis: Union[Dim, Sequence[Dim]]):
        norm = normalize(a, axis=axis, epsilon=self.epsilon)
        if self.scale is not None:
            norm = self.scale * norm
        if self.bias is not None:
            norm = norm + self.bias
        return norm


def batch_norm_distributed_default() -> bool:
    """config option ``rf_batch_norm_distributed`` (default False): batch-norm statistics summed over all data-parallel ranks"""
    from ..config import get_global_config

    config = get_global_config(raise_exception=False)
    return bool(config.bool("rf_batch_norm_distributed", False)) if config else False
