"""
Convolution, transposed convolution and pooling over named spatial dims.

"same" padding: total padding is ``k - 1 - (in_len - 1) % stride`` per spatial dim, the smaller half on the left, so that
``out_len = ceil(in_len / stride)`` and the first and last window see the same amount of padding (up to one frame).

Parity: returnn/frontend/conv.py:260-740; returnn/torch/frontend/_backend.py:2336-2466 (conv), :2567-2631 (pool).
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union, List
import torch
import torch.nn.functional as F
from ..tensor import Tensor, Dim
from .module import Module
from .parameter import Parameter
from . import init as _init
from ._utils import wrap, axis_of

__all__ = ["conv", "Conv1d", "Conv2d", "Conv3d", "transposed_conv", "TransposedConv1d", "TransposedConv2d",
           "TransposedConv3d", "pool", "max_pool", "max_pool1d", "pool1d", "pool2d", "pool3d", "make_conv_out_spatial_dims",
           "calc_conv_out_spatial_length", "calc_conv_out_length", "calc_transposed_conv_out_length",
           "make_transposed_conv_out_spatial_dims"]


def _tup(v, n) -> Tuple[int, ...]:
    if v is None:
        return (1,) * n
    if isinstance(v, int):
        return (v,) * n
    assert len(v) == n
    return tuple(int(x) for x in v)


def calc_conv_out_spatial_length(in_len, *, filter_size: int, stride: int = 1, dilation_rate: int = 1, padding: Union[str, int] = "valid"):
    """output length of one spatial dim (int or tensor)"""
    if isinstance(padding, str) and padding.lower() == "same":
        return -(-in_len // stride)
    if isinstance(padding, str):
        assert padding.lower() == "valid"
        eff = in_len - (filter_size - 1) * dilation_rate
    else:
        eff = in_len + 2 * padding - (filter_size - 1) * dilation_rate
    return -(-eff // stride)


def make_conv_out_spatial_dims(in_spatial_dims: Sequence[Dim], *, filter_size, padding, strides=1, dilation_rate=1,
                               description_prefix: Optional[str] = None) -> List[Dim]:
    """out spatial dims (derived dims; their sizes follow the input sizes)"""
    n = len(in_spatial_dims)
    fs = tuple(f.dimension if isinstance(f, Dim) else f for f in (filter_size if isinstance(filter_size, (list, tuple)) else [filter_size] * n))
    st, dl = _tup(strides, n), _tup(dilation_rate, n)
    pads = [padding] * n if isinstance(padding, (str, int)) else list(padding)
    out = []
    for i, d in enumerate(in_spatial_dims):
        p = pads[i].lower() if isinstance(pads[i], str) else pads[i]
        if p == "same" and st[i] == 1:
            out.append(d)
        elif p == "same":
            out.append(d.ceildiv_right(st[i]))
        elif fs[i] == 1 and st[i] == 1 and p in ("valid", 0):
            out.append(d)
        else:
            out.append(Dim._derive("conv", [d], attribs={"filter_size": fs[i], "stride": st[i], "dilation": dl[i], "padding": p}))
    return out


def _mask_input(source: Tensor, in_spatial_dims: Sequence[Dim], use_mask: Optional[bool]) -> Tensor:
    if use_mask is None:
        from .dims import use_mask_default

        use_mask = use_mask_default(default=True, default_false_for_behavior_version_up_to=22)
    if use_mask:
        for d in in_spatial_dims:
            if d.is_dynamic() and d.need_masking() and d.is_dynamic_seq_length():
                source = source.copy_masked(0, dims=[d])
    return source


def _use_consistent_same_padding() -> bool:
    """
    Whether ``padding="same"`` with a stride pads by ``(filter_size - 1) / 2`` on both sides whatever the length (behaviour
    version >= 24, or the config option ``rf_use_consistent_same_padding``), instead of the TensorFlow rule whose padding depends on
    the padded length of the batch: with that rule a sequence's frames see a different alignment of the windows depending on the
    longest sequence it happens to be batched with. Reference: returnn/frontend/conv.py:1019-1048.
    """
    from ..config import get_global_config
    from ..utils.basic import BehaviorVersion

    config = get_global_config(raise_exception=False)
    if config is not None:
        if "rf_use_consistent_same_padding" in config.typed_dict:
            v = config.typed_dict["rf_use_consistent_same_padding"]
            if v is not None:
                return bool(v)
        elif "rf_use_consistent_same_padding" in config.dict:
            v = config.bool("rf_use_consistent_same_padding", None)
            if v is not None:
                return v
    return BehaviorVersion.get() >= 24


def _same_pads(shape_spatial, fs, st) -> List[int]:
    """``F.pad`` argument (last axis first) for "same" padding; ``fs``: effective (dilated) filter sizes"""
    consistent = any(s != 1 for s in st) and _use_consistent_same_padding()
    pads: List[int] = []
    for i in reversed(range(len(fs))):
        if consistent:
            pad = fs[i] - 1
        else:
            pad = max(fs[i] - 1 - (shape_spatial[i] - 1) % st[i], 0)
        left = pad // 2
        pads.extend([left, pad - left])
    return pads


def conv(source: Tensor, *, in_dim: Dim, out_dim: Dim, in_spatial_dims: Sequence[Dim],
         out_spatial_dims: Optional[Sequence[Dim]] = None, filter: Tensor, filter_size: Sequence[Dim],
         padding: Union[str, int, Sequence[int]], strides=None, dilation_rate=None, groups: Optional[int] = None,
         bias: Optional[Tensor] = None, use_mask: Optional[bool] = None) -> Tuple[Tensor, Sequence[Dim]]:
    """
    N-d convolution (N = 1, 2, 3). filter dims: ``(out_dim, in_dim // groups, *filter_size)``.
    """
    n = len(in_spatial_dims)
    if n == 1 and in_spatial_dims[0] not in source._dims:
        from . import packed_mode

        pdim = packed_mode.packed_dim_of(source, in_spatial_dims[0])
        if pdim is not None:  # packed rows: no padded frames exist, so nothing to mask; run on the padded form and pack the result
            return packed_mode.apply_padded(
                lambda padded: conv(padded, in_dim=in_dim, out_dim=out_dim, in_spatial_dims=in_spatial_dims, out_spatial_dims=out_spatial_dims,
                                    filter=filter, filter_size=filter_size, padding=padding, strides=strides, dilation_rate=dilation_rate, groups=groups,
                                    bias=bias, use_mask=use_mask), source, pdim)
    source = _mask_input(source, in_spatial_dims, use_mask)
    if not out_spatial_dims:
        out_spatial_dims = make_conv_out_spatial_dims(in_spatial_dims, filter_size=filter_size, strides=strides or 1,
                                                      dilation_rate=dilation_rate or 1, padding=padding)
    fs = tuple(f.dimension for f in filter_size)
    st, dl = _tup(strides, n), _tup(dilation_rate, n)
    batch_dims = [d for d in source._dims if d != in_dim and d not in in_spatial_dims]
    raw = source.copy_compatible_to_dims_raw(batch_dims + [in_dim] + list(in_spatial_dims))
    bshape = list(raw.shape[: len(batch_dims)])
    raw = raw.reshape([-1] + list(raw.shape[len(batch_dims):]))
    w = filter._raw_tensor
    if filter._dims[0] != out_dim:
        w = filter.copy_compatible_to_dims_raw([out_dim, filter._dims[[i for i, d in enumerate(filter._dims) if d not in filter_size and d != out_dim][0]]] + list(filter_size))
    pad_arg: Union[int, Tuple[int, ...]]
    if isinstance(padding, str) and padding.lower() == "same":
        pads = _same_pads(raw.shape[2:], tuple((f - 1) * d + 1 for f, d in zip(fs, dl)), st)
        if any(pads):
            raw = F.pad(raw, pads)
        pad_arg = 0
    elif isinstance(padding, str):
        assert padding.lower() == "valid"
        pad_arg = 0
    else:
        pad_arg = padding if isinstance(padding, int) else tuple(padding)
    b = bias._raw_tensor if bias is not None else None
    if w.dtype != raw.dtype and not torch.is_autocast_enabled():
        w = w.to(raw.dtype)
        b = b.to(raw.dtype) if b is not None else None
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[n]
    out = fn(raw, w, b, stride=st, padding=pad_arg, dilation=dl, groups=groups or 1)
    out = out.reshape(bshape + list(out.shape[1:]))
    res = wrap(out, batch_dims + [out_dim] + list(out_spatial_dims), feature_dim=out_dim)
    return res, out_spatial_dims


class _ConvNd(Module):
    nd: int = 0

    def __init__(self, in_dim: Dim, out_dim: Dim, filter_size, *, padding: Union[str, int, Sequence[int]], strides=None,
                 dilation_rate=None, groups: Optional[int] = None, with_bias: bool = True):
        super().__init__()
        assert isinstance(in_dim, Dim) and isinstance(out_dim, Dim)
        self.in_dim = in_dim
        self.out_dim = out_dim
        if isinstance(filter_size, (int, Dim)):
            filter_size = [filter_size] * self.nd
        assert len(filter_size) == self.nd
        self.filter_size = [s if isinstance(s, Dim) else Dim(s, name="filter-dim%i" % i) for i, s in enumerate(filter_size)]
        self.padding = padding
        self.strides = strides
        self.dilation_rate = dilation_rate
        self.groups = groups
        self.filter_in_dim = in_dim if not groups or groups == 1 else in_dim // groups
        self.filter = Parameter([out_dim, self.filter_in_dim] + self.filter_size)
        self.filter.initial = _init.Glorot()
        self.with_bias = with_bias
        self.bias = None
        if with_bias:
            self.bias = Parameter([out_dim])
            self.bias.initial = 0.0

    def _call_nd(self, source: Tensor, in_spatial_dims, out_spatial_dims=None):
        return conv(source, in_dim=self.in_dim, out_dim=self.out_dim, in_spatial_dims=in_spatial_dims,
                    out_spatial_dims=out_spatial_dims, filter=self.filter, filter_size=self.filter_size,
                    padding=self.padding, strides=self.strides, dilation_rate=self.dilation_rate, groups=self.groups,
                    bias=self.bias)


class Conv1d(_ConvNd):
    """1-D convolution"""

    nd = 1

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim, out_spatial_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
        out, (osd,) = self._call_nd(source, [in_spatial_dim], [out_spatial_dim] if out_spatial_dim else None)
        return out, osd


class Conv2d(_ConvNd):
    """2-D convolution"""

    nd = 2

    def __call__(self, source: Tensor, *, in_spatial_dims: Sequence[Dim], out_spatial_dims: Optional[Sequence[Dim]] = None):
        assert len(in_spatial_dims) == 2
        return self._call_nd(source, in_spatial_dims, out_spatial_dims)


class Conv3d(_ConvNd):
    """3-D convolution"""

    nd = 3

    def __call__(self, source: Tensor, *, in_spatial_dims: Sequence[Dim], out_spatial_dims: Optional[Sequence[Dim]] = None):
        assert len(in_spatial_dims) == 3
        return self._call_nd(source, in_spatial_dims, out_spatial_dims)


def transposed_conv(source: Tensor, *, in_dim: Dim, out_dim: Dim, in_spatial_dims: Sequence[Dim],
                    out_spatial_dims: Optional[Sequence[Dim]] = None, filter: Tensor, filter_size: Sequence[Dim],
                    padding: str, remove_padding: Union[Sequence[int], int] = 0, output_padding=None,
                    strides: Optional[Sequence[int]] = None, bias: Optional[Tensor] = None, use_mask: Optional[bool] = None):
    """transposed (fractionally strided) convolution; filter dims ``(in_dim, out_dim, *filter_size)``"""
    n = len(in_spatial_dims)
    source = _mask_input(source, in_spatial_dims, use_mask)
    fs = tuple(f.dimension for f in filter_size)
    st = _tup(strides if strides is not None else fs, n)
    rp = _tup(remove_padding, n)
    op = _tup(output_padding if output_padding is not None else 0, n)
    batch_dims = [d for d in source._dims if d != in_dim and d not in in_spatial_dims]
    raw = source.copy_compatible_to_dims_raw(batch_dims + [in_dim] + list(in_spatial_dims))
    bshape = list(raw.shape[: len(batch_dims)])
    raw = raw.reshape([-1] + list(raw.shape[len(batch_dims):]))
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[n]
    w = filter._raw_tensor
    if w.dtype != raw.dtype and not torch.is_autocast_enabled():
        w = w.to(raw.dtype)
    out = fn(raw, w, bias._raw_tensor if bias is not None else None, stride=st, output_padding=op)
    if padding.lower() == "same":
        # cut so that out_len = in_len * stride
        for i in range(n):
            want = raw.shape[2 + i] * st[i]
            extra = out.shape[2 + i] - want
            if extra > 0:
                out = out.narrow(2 + i, extra // 2, want)
    for i in range(n):
        if rp[i]:
            out = out.narrow(2 + i, rp[i], out.shape[2 + i] - 2 * rp[i])
    if not out_spatial_dims:
        out_spatial_dims = []
        for i, d in enumerate(in_spatial_dims):
            od = d * st[i]
            if padding.lower() != "same":
                extra = max(fs[i] - st[i], 0) + op[i] - 2 * rp[i]
                od = od + extra if extra else od
            elif rp[i]:
                od = od - 2 * rp[i]
            out_spatial_dims.append(od)
    out = out.reshape(bshape + list(out.shape[1:]))
    return wrap(out, batch_dims + [out_dim] + list(out_spatial_dims), feature_dim=out_dim), out_spatial_dims


class _TransposedConvNd(Module):
    nd: int = 0

    def __init__(self, in_dim: Dim, out_dim: Dim, filter_size, *, padding: str = "valid", remove_padding=0,
                 output_padding=None, strides=None, with_bias: bool = True):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        if isinstance(filter_size, (int, Dim)):
            filter_size = [filter_size] * self.nd
        self.filter_size = [s if isinstance(s, Dim) else Dim(s, name="filter-dim%i" % i) for i, s in enumerate(filter_size)]
        self.strides = strides
        self.padding = padding
        self.remove_padding = remove_padding
        self.output_padding = output_padding
        self.filter = Parameter([in_dim, out_dim] + self.filter_size)
        self.filter.initial = _init.Glorot()
        self.with_bias = with_bias
        self.bias = None
        if with_bias:
            self.bias = Parameter([out_dim])
            self.bias.initial = 0.0

    def _call_nd(self, source, in_spatial_dims, out_spatial_dims=None):
        return transposed_conv(source, in_dim=self.in_dim, out_dim=self.out_dim, in_spatial_dims=in_spatial_dims,
                               out_spatial_dims=out_spatial_dims, filter=self.filter, filter_size=self.filter_size,
                               padding=self.padding, remove_padding=self.remove_padding, output_padding=self.output_padding,
                               strides=self.strides, bias=self.bias)


class TransposedConv1d(_TransposedConvNd):
    """1-D transposed conv"""

    nd = 1

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim, out_spatial_dim: Optional[Dim] = None):
        out, (osd,) = self._call_nd(source, [in_spatial_dim], [out_spatial_dim] if out_spatial_dim else None)
        return out, osd


class TransposedConv2d(_TransposedConvNd):
    """2-D transposed conv"""

    nd = 2

    def __call__(self, source, *, in_spatial_dims, out_spatial_dims=None):
        return self._call_nd(source, in_spatial_dims, out_spatial_dims)


class TransposedConv3d(_TransposedConvNd):
    """3-D transposed conv"""

    nd = 3

    def __call__(self, source, *, in_spatial_dims, out_spatial_dims=None):
        return self._call_nd(source, in_spatial_dims, out_spatial_dims)


def pool(source: Tensor, *, mode: str, pool_size: Union[Sequence[int], int], padding: Union[Sequence[str], str, Sequence[int], int] = "valid",
         dilation_rate=1, strides=None, in_spatial_dims: Union[Sequence[Dim], Dim],
         out_spatial_dims: Optional[Union[Sequence[Dim], Dim]] = None, use_mask: Optional[bool] = None):
    """
    max / avg pooling over the spatial dims. Padded frames count as ``-inf`` (max) or are left out of the mean (avg).
    """
    if isinstance(in_spatial_dims, Dim):
        in_spatial_dims = [in_spatial_dims]
    n = len(in_spatial_dims)
    if n == 1 and in_spatial_dims[0] not in source._dims:
        from . import packed_mode

        pdim = packed_mode.packed_dim_of(source, in_spatial_dims[0])
        if pdim is not None:
            return packed_mode.apply_padded(
                lambda padded: pool(padded, mode=mode, pool_size=pool_size, padding=padding, dilation_rate=dilation_rate, strides=strides,
                                    in_spatial_dims=in_spatial_dims, out_spatial_dims=out_spatial_dims, use_mask=use_mask), source, pdim)
    ps = _tup(pool_size, n)
    st = _tup(strides if strides is not None else ps, n)
    dl = _tup(dilation_rate, n)
    mode = mode.lower()
    if mode == "average":
        mode = "avg"
    assert mode in ("max", "avg")
    if use_mask is None:
        from .dims import use_mask_default

        use_mask = use_mask_default(default=True, default_false_for_behavior_version_up_to=22)
    if use_mask:
        for d in in_spatial_dims:
            if d.is_dynamic() and d.need_masking() and d.is_dynamic_seq_length():
                source = source.copy_masked(float("-inf") if mode == "max" else 0, dims=[d])
    if out_spatial_dims is None:
        out_spatial_dims = make_conv_out_spatial_dims(in_spatial_dims, filter_size=ps, strides=st, dilation_rate=dl, padding=padding)
    elif isinstance(out_spatial_dims, Dim):
        out_spatial_dims = [out_spatial_dims]
    other = [d for d in source._dims if d not in in_spatial_dims]
    raw = source.copy_compatible_to_dims_raw(other + list(in_spatial_dims))
    oshape = list(raw.shape[: len(other)])
    raw = raw.reshape([1, -1] + list(raw.shape[len(other):]))
    if isinstance(padding, str) and padding.lower() == "same":
        pads = _same_pads(raw.shape[2:], tuple((f - 1) * d + 1 for f, d in zip(ps, dl)), st)
        if any(pads):
            raw = F.pad(raw, pads, value=float("-inf") if mode == "max" else 0.0)
        pad_arg: Union[int, Tuple[int, ...]] = 0
    elif isinstance(padding, str):
        pad_arg = 0
    else:
        pad_arg = padding if isinstance(padding, int) else tuple(padding)
    if mode == "max":
        fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[n]
        out = fn(raw, kernel_size=ps, stride=st, padding=pad_arg, dilation=dl)
    else:
        fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[n]
        out = fn(raw, kernel_size=ps, stride=st, padding=pad_arg)
    out = out.reshape(oshape + list(out.shape[2:]))
    res = wrap(out, other + list(out_spatial_dims), like=source)
    if mode == "max" and use_mask:
        res = res.copy_masked(0)
    return res, out_spatial_dims


def max_pool(source, *, pool_size, padding="valid", dilation_rate=1, strides=None, in_spatial_dims, out_spatial_dims=None):
    """max pooling"""
    return pool(source, mode="max", pool_size=pool_size, padding=padding, dilation_rate=dilation_rate, strides=strides,
                in_spatial_dims=in_spatial_dims, out_spatial_dims=out_spatial_dims)


def max_pool1d(source, *, pool_size: int, padding="valid", dilation_rate=1, strides=None, in_spatial_dim: Dim, out_spatial_dim=None):
    """1-D max pooling"""
    return pool1d(source, mode="max", pool_size=pool_size, padding=padding, dilation_rate=dilation_rate, strides=strides,
                  in_spatial_dim=in_spatial_dim, out_spatial_dim=out_spatial_dim)


def pool1d(source, *, mode: str, pool_size: int, padding="valid", dilation_rate=1, strides=None, in_spatial_dim: Dim, out_spatial_dim=None):
    """1-D pooling"""
    res, (osd,) = pool(source, mode=mode, pool_size=[pool_size], padding=padding, dilation_rate=dilation_rate,
                       strides=[strides] if isinstance(strides, int) else strides, in_spatial_dims=[in_spatial_dim],
                       out_spatial_dims=[out_spatial_dim] if out_spatial_dim is not None else None)
    return res, osd


def pool2d(source, *, mode, pool_size, padding="valid", dilation_rate=1, strides=None, in_spatial_dims, out_spatial_dims=None):
    """2-D pooling"""
    return pool(source, mode=mode, pool_size=pool_size, padding=padding, dilation_rate=dilation_rate, strides=strides,
                in_spatial_dims=in_spatial_dims, out_spatial_dims=out_spatial_dims)


def pool3d(source, *, mode, pool_size, padding="valid", dilation_rate=1, strides=None, in_spatial_dims, out_spatial_dims=None):
    """3-D pooling"""
    return pool(source, mode=mode, pool_size=pool_size, padding=padding, dilation_rate=dilation_rate, strides=strides,
                in_spatial_dims=in_spatial_dims, out_spatial_dims=out_spatial_dims)


def calc_conv_out_length(in_length, *, filter_size, stride: int, padding: Union[str, int], dilation_rate: int = 1, name: Optional[str] = None):
    """
    Output length of a convolution along one axis, for an int, a size tensor or a :class:`Dim` (then a derived Dim whose sequence
    lengths follow the input's).  "same": ``ceil(n / stride)``; "valid" or an int padding: ``ceil((n + 2p - (k - 1) d) / stride)``.
    Reference: returnn/frontend/conv.py:783-858.
    """
    k = filter_size.dimension if isinstance(filter_size, Dim) else filter_size
    pad = padding.lower() if isinstance(padding, str) else padding
    if isinstance(in_length, Dim):
        out = make_conv_out_spatial_dims([in_length], filter_size=[k], padding=pad, strides=stride, dilation_rate=dilation_rate)[0]
        if name and out is not in_length:
            out.name = name
        return out
    if (k == stride == 1 and pad in ("valid", "same", 0)) or (stride == 1 and pad == "same"):
        return in_length
    if isinstance(in_length, Tensor):
        raw = calc_conv_out_spatial_length(in_length.raw_tensor, filter_size=k, stride=stride, dilation_rate=dilation_rate, padding=pad)
        return in_length.copy_with_raw(torch.clamp(raw, min=0) if isinstance(raw, torch.Tensor) else raw)
    return max(calc_conv_out_spatial_length(in_length, filter_size=k, stride=stride, dilation_rate=dilation_rate, padding=pad), 0)


def calc_transposed_conv_out_length(in_length, *, filter_size, padding: Union[int, str], output_padding: Optional[int] = None,
                                    stride: Optional[int] = None, dilation_rate: int = 1, name: Optional[str] = None):
    """
    Output length of a transposed convolution along one axis (int, size tensor or Dim): ``n * stride`` plus, for "valid",
    ``max(k - stride, 0)``; "same": ``n * stride``; "full": ``n * stride - (stride + k - 2)``; with ``output_padding`` the exact
    ``n * stride + k - stride - 2 * pad + output_padding``.  Reference: returnn/frontend/conv.py:910-1004.
    """
    assert padding in ("same", "valid", "full") or isinstance(padding, int)
    k = filter_size.dimension if isinstance(filter_size, Dim) else filter_size
    if dilation_rate != 1 and k != 1:
        k = k + (k - 1) * (dilation_rate - 1)
    if stride is None:
        stride = k

    def calc(n):
        n = n * stride if stride != 1 else n
        if output_padding is None:
            if padding == "valid" or padding == 0:
                return n if k == stride else n + max(k - stride, 0)
            if padding == "full":
                return n - (stride + k - 2)
            if padding == "same":
                return n
            raise ValueError("calc_transposed_conv_out_length: invalid padding %r without output_padding" % (padding,))
        pad = {"same": k // 2, "valid": 0, "full": k - 1}.get(padding, padding)
        return n + (k - stride - 2 * pad + output_padding)

    if isinstance(in_length, Dim):
        if in_length.dimension is not None:
            out = Dim(calc(in_length.dimension), name=name or ("%s:transposed-conv" % (in_length.name or "dim")))
        else:
            out = Dim(None, name=name or ("%s:transposed-conv" % (in_length.name or "dim")))
            if in_length.dyn_size_ext is not None:
                out.dyn_size_ext = in_length.dyn_size_ext.copy_with_raw(calc(in_length.dyn_size_ext.raw_tensor))
        return out
    if isinstance(in_length, Tensor):
        return in_length.copy_with_raw(calc(in_length.raw_tensor))
    return calc(in_length)


def make_transposed_conv_out_spatial_dims(in_spatial_dims: Sequence[Dim], *, filter_size, padding, output_padding=None, strides=None,
                                          dilation_rate=1, description_prefix: Optional[str] = None) -> List[Dim]:
    """out spatial dims of a transposed convolution, one per in spatial dim (see :func:`calc_transposed_conv_out_length`)"""
    n = len(in_spatial_dims)

    def seq(v):
        return list(v) if isinstance(v, (list, tuple)) else [v] * n

    fs = [d.dimension if isinstance(d, Dim) else d for d in seq(filter_size)]
    st, dl, pd, op = seq(strides), seq(dilation_rate), seq(padding), seq(output_padding)
    return [calc_transposed_conv_out_length(in_spatial_dims[i], filter_size=fs[i], padding=pd[i].lower() if isinstance(pd[i], str) else pd[i],
                                            output_padding=op[i], stride=st[i], dilation_rate=dl[i],
                                            name="%s:spatial%i" % (description_prefix, i) if description_prefix else None) for i in range(n)]
