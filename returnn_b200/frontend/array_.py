"""
Array ops on named-dim tensors: reshape-like (merge/split dims), concat/pad/stack, gather/scatter, masking and
packing, slicing and shifting, sort, top-k / top-p masks.

Parity: returnn/frontend/array_.py:1-1624.
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union, List, Any, Dict
import numpy
import torch
import torch.nn.functional as F
from ..tensor import Tensor, Dim, batch_dim
from ..utils.basic import NotSpecified
from ._utils import wrap, convert_to_tensor as _convert_to_tensor, torch_dtype, dtype_name, axis_of, merge_dims_for_broadcast

__all__ = [
    "convert_to_tensor", "constant_value", "copy", "cast", "merge_dims", "split_dims", "reshape", "split", "expand_dim",
    "expand_dims", "squeeze", "window", "concat", "concat_features", "pad", "cum_concat_step", "stack", "masked_select",
    "masked_scatter", "sequence_mask", "pack_padded", "gather", "scatter", "scatter_mean", "scatter_argmax",
    "scatter_logsumexp", "scatter_logmeanexp", "slice", "shift_right", "shift_left", "reverse_sequence", "where",
    "search_sorted", "sparse_to_dense", "one_hot", "top_k_mask", "top_p_mask", "sort", "repeat", "tile", "cumsum",
    "transpose", "num_elements_of_shape", "is_true", "nonzero_indices", "unstack", "scatter_count", "pad_packed",
    "expand_make_non_empty", "real_as_complex", "complex_as_real", "make_complex",
]


def convert_to_tensor(value, *, dims: Sequence[Dim] = (), dtype: Optional[str] = None, sparse_dim: Optional[Dim] = None,
                      feature_dim: Optional[Dim] = None, shape: Optional[Sequence[Dim]] = None, device: Optional[str] = None,
                      keep_scalar_on_cpu: bool = False, name: Optional[str] = None, _backend=None) -> Tensor:
    """python / numpy / torch value -> Tensor"""
    if shape is not None and not dims:
        dims = shape
    if device is None and not keep_scalar_on_cpu:
        from .device import get_default_device

        device = get_default_device()
    if keep_scalar_on_cpu and not dims:
        device = "cpu"
    return _convert_to_tensor(value, dims=dims, dtype=dtype, sparse_dim=sparse_dim, feature_dim=feature_dim, device=device, name=name)


def constant_value(x: Tensor):
    """python value if x is a known constant scalar on the host"""
    if x._raw_tensor is not None and not x._dims and x._raw_tensor.device.type == "cpu":
        return x._raw_tensor.item()
    return None


def is_true(x: Tensor) -> bool:
    """host bool of a scalar"""
    return bool(x._raw_tensor)


def copy(x: Tensor) -> Tensor:
    """identity (new Tensor object, same storage)"""
    return x.copy()


def cast(x: Tensor, dtype: str) -> Tensor:
    """dtype conversion"""
    if x.dtype == dtype:
        return x
    return wrap(x._raw_tensor.to(torch_dtype(dtype)), x._dims, like=x)


def transpose(x: Tensor, perm: Sequence[Dim]) -> Tensor:
    """reorder axes"""
    return x.copy_transpose_to_dims(perm)


def num_elements_of_shape(dims: Union[Dim, Sequence[Dim]], *, use_mask: bool = True, device: Optional[str] = None) -> Union[int, Tensor]:
    """number of (non-padded) elements in a shape"""
    if isinstance(dims, Dim):
        dims = [dims]
    n: Any = 1
    remaining = list(dims)  # a static dim may occur more than once (a square weight matrix): every occurrence counts
    # dynamic dims with sizes over other dims in the list: sum of sizes, which accounts for those other dims too
    for d in list(remaining):
        if d not in remaining:
            continue
        if d.is_dynamic() and not d.is_batch_dim() and use_mask and d.dyn_size_ext is not None and d.dyn_size_ext.dims:
            ext = d.dyn_size_ext
            assert all(dd in dims for dd in ext.dims), "num_elements_of_shape: %r sizes depend on dims outside %r" % (d, dims)
            total = ext.raw_tensor.sum()
            # lengths on the device (static-shape / CUDA-graph regime): stay on the device, the count becomes a scalar Tensor
            n = n * (total if getattr(total, "is_cuda", False) else int(total))
            remaining.remove(d)
            for dd in ext.dims:
                if dd in remaining:
                    remaining.remove(dd)
    for d in remaining:
        n = n * d.get_dim_value()
    if isinstance(n, torch.Tensor):
        return Tensor("num_elements", dims=[], dtype=dtype_name(n.dtype), raw_tensor=n)
    return n


def merge_dims(source: Tensor, *, dims: Sequence[Dim], out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    Flatten several axes into one (row-major in the order of ``dims``). The merged axis sits where the first one was.
    Padding stays inside; the new dim has no per-sequence sizes.
    """
    dims = list(dims)
    if not dims:
        if out_dim is None:
            out_dim = Dim(1, name="ext")
        return expand_dim(source, out_dim), out_dim
    if len(dims) == 1:
        if out_dim is None or out_dim == dims[0]:
            return source, dims[0]
    if out_dim is None:
        out_dim = dims[0]
        for d in dims[1:]:
            out_dim = out_dim * d
    axes = [axis_of(source, d) for d in dims]
    first = min(axes)
    rest = [i for i in range(len(source._dims)) if i not in axes]
    perm = rest[:first] + axes + rest[first:]
    # `first` counts position among all axes; number of rest axes before it:
    n_before = len([i for i in rest if i < first])
    perm = rest[:n_before] + axes + rest[n_before:]
    raw = source._raw_tensor.permute(*perm)
    shape = list(raw.shape)
    merged = 1
    for s in shape[n_before : n_before + len(axes)]:
        merged *= s
    new_shape = shape[:n_before] + [merged] + shape[n_before + len(axes):]
    raw = raw.reshape(new_shape)
    out_dims = [source._dims[i] for i in rest[:n_before]] + [out_dim] + [source._dims[i] for i in rest[n_before:]]
    if out_dim.is_dynamic() and out_dim.dyn_size_ext is None:
        out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=[], dtype="int32", raw_tensor=torch.tensor(merged, dtype=torch.int32))
    fd = None
    if source.feature_dim is not None and source.feature_dim in dims:
        fd = out_dim
    res = wrap(raw, out_dims, like=source)
    if fd is not None:
        res._feature_dim = fd
    return res, out_dim


def split_dims(source: Tensor, *, axis: Dim, dims: Sequence[Dim], pad_to_multiples=None, pad_value=None) -> Tensor:
    """unflatten ``axis`` into ``dims``"""
    ax = axis_of(source, axis)
    raw = source._raw_tensor
    sizes = []
    unknown = None
    for i, d in enumerate(dims):
        if d.is_static():
            sizes.append(d.dimension)
        else:
            try:
                sizes.append(d.get_dim_value())
            except Exception:
                sizes.append(-1)
                assert unknown is None
                unknown = i
    new_shape = list(raw.shape[:ax]) + sizes + list(raw.shape[ax + 1:])
    raw = raw.reshape(new_shape)
    out_dims = list(source._dims[:ax]) + list(dims) + list(source._dims[ax + 1:])
    if unknown is not None:
        d = dims[unknown]
        d.dyn_size_ext = Tensor("%s:size" % d.name, dims=[], dtype="int32", raw_tensor=torch.tensor(raw.shape[ax + unknown], dtype=torch.int32))
    res = wrap(raw, out_dims, like=source)
    if source.feature_dim == axis:
        res._feature_dim = dims[-1]
    return res


def reshape(source: Tensor, in_dims: Sequence[Dim], out_dims: Sequence[Dim]) -> Tensor:
    """general reshape of a contiguous group of dims"""
    merged, md = merge_dims(source, dims=in_dims)
    return split_dims(merged, axis=md, dims=out_dims)


def split(source: Tensor, *, axis: Dim, out_dims: Sequence[Dim]) -> Tuple[Tensor, ...]:
    """split along axis into parts of the given dims"""
    ax = axis_of(source, axis)
    sizes = [d.get_dim_value() for d in out_dims]
    parts = torch.split(source._raw_tensor, sizes, dim=ax)
    res = []
    for p, d in zip(parts, out_dims):
        dims = list(source._dims)
        dims[ax] = d
        t = wrap(p, dims, like=source)
        if source.feature_dim == axis:
            t._feature_dim = d
        res.append(t)
    return tuple(res)


def expand_dim(source: Tensor, dim: Dim) -> Tensor:
    """add an axis (broadcast) at the end, or before the feature dim for spatial dims"""
    if dim.is_static() and dim.dimension == 1:
        return wrap(source._raw_tensor.unsqueeze(-1), list(source._dims) + [dim], like=source)
    raw = source._raw_tensor.unsqueeze(-1)
    shape = list(raw.shape)
    shape[-1] = dim.get_dim_value()
    return wrap(raw.expand(*shape), list(source._dims) + [dim], like=source)


def expand_dims(source: Tensor, dims: Sequence[Dim]) -> Tensor:
    """add several axes"""
    for d in dims:
        source = expand_dim(source, d)
    return source


def squeeze(source: Tensor, axis: Dim) -> Tensor:
    """remove a size-1 axis"""
    ax = axis_of(source, axis)
    assert source._raw_tensor.shape[ax] == 1
    dims = list(source._dims)
    dims.pop(ax)
    return wrap(source._raw_tensor.squeeze(ax), dims, like=source)


def window(source: Tensor, *, spatial_dim: Dim, window_dim: Dim, window_right: Optional[int] = None,
           window_left: Optional[int] = None, padding: str = "same", pad_value=None, stride: int = 1,
           use_mask: Optional[bool] = None) -> Tuple[Tensor, Dim]:
    """
    Sliding windows over spatial_dim: out[..., t, w, ...] = source[..., t*stride + w - left, ...].
    :return: out with window_dim inserted after spatial_dim, out spatial dim
    """
    assert window_dim.is_static()
    w = window_dim.dimension
    if window_left is None and window_right is None:
        window_right = w // 2
        window_left = w - window_right - 1
    elif window_left is None:
        window_left = w - window_right - 1
    elif window_right is None:
        window_right = w - window_left - 1
    if use_mask is None:
        use_mask = True
    if use_mask and spatial_dim.is_dynamic() and spatial_dim.is_dynamic_seq_length():
        source = source.copy_masked(0 if pad_value is None else pad_value, dims=[spatial_dim])
    ax = axis_of(source, spatial_dim)
    raw = source._raw_tensor
    if padding == "same":
        pad = [0, 0] * (raw.ndim - ax - 1) + [window_left, window_right]
        raw = F.pad(raw, pad, value=0 if pad_value is None else pad_value)
        out_spatial = spatial_dim if stride == 1 else spatial_dim.ceildiv_right(stride)
    elif padding == "valid":
        out_spatial = Dim._derive("conv", [spatial_dim], attribs={"filter_size": w, "stride": stride, "dilation": 1, "padding": "valid"})
    else:
        raise ValueError("window: invalid padding %r" % (padding,))
    raw = raw.unfold(ax, w, stride)  # window axis is last
    raw = raw.movedim(-1, ax + 1)
    dims = list(source._dims[: ax]) + [out_spatial, window_dim] + list(source._dims[ax + 1:])
    return wrap(raw, dims, like=source), out_spatial


def concat(*sources: Tuple[Tensor, Dim], allow_broadcast: bool = False, out_dim: Optional[Dim] = None,
           handle_dynamic_dims: Optional[bool] = None) -> Tuple[Tensor, Dim]:
    """
    Concatenate ``(tensor, dim)`` pairs along their dims.
    When a concat dim has per-sequence sizes, the valid frames of each sequence are made contiguous.
    """
    assert sources
    if out_dim is None:
        out_dim = sources[0][1]
        for _, d in sources[1:]:
            out_dim = out_dim + d
    need_dyn = any(d.is_dynamic() and d.is_dynamic_seq_length() for _, d in sources[:-1])
    if handle_dynamic_dims is None:
        handle_dynamic_dims = True
    first, first_dim = sources[0]
    ref_dims = [d for d in first._dims if d != first_dim]
    all_other: List[Dim] = list(ref_dims)
    for t, d in sources[1:]:
        for dd in t._dims:
            if dd != d and dd not in all_other:
                assert allow_broadcast, "concat: %r has extra dim %r; set allow_broadcast" % (t, dd)
                all_other.append(dd)
    ax0 = axis_of(first, first_dim)
    template = list(all_other)
    pos = min(ax0, len(template))
    raws = []
    for t, d in sources:
        tgt = template[:pos] + [d] + template[pos:]
        r = t.copy_compatible_to_dims_raw(tgt)
        shape = [dd.get_dim_value() if dd != d else r.shape[i] for i, dd in enumerate(tgt)]
        if list(r.shape) != shape:
            r = r.expand(*shape)
        raws.append(r)
    out_dims = template[:pos] + [out_dim] + template[pos:]
    if need_dyn and handle_dynamic_dims:
        # place each part at its per-sequence offset
        total_sizes = None
        for _, d in sources:
            s = d.get_size_tensor() if d.is_dynamic() else None
            sz = s.copy_compatible_to_dims_raw([batch_dim]).to(torch.int64) if (s is not None and s.dims) else torch.tensor(d.get_dim_value(), dtype=torch.int64)
            total_sizes = sz if total_sizes is None else total_sizes + sz
        if out_dim.dyn_size_ext is None:
            out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=[batch_dim], dtype="int32", raw_tensor=total_sizes.to(torch.int32))
        max_len = int(total_sizes.max())
        bax = out_dims.index(batch_dim)
        device = raws[0].device
        out_shape = list(raws[0].shape)
        out_shape[pos] = max_len
        out = torch.zeros(out_shape, dtype=raws[0].dtype, device=device)
        offsets = torch.zeros_like(total_sizes.reshape(-1) if total_sizes.ndim else total_sizes.expand(out_shape[bax]))
        offsets = offsets.to(device)
        for (t, d), r in zip(sources, raws):
            n = r.shape[pos]
            s = d.get_size_tensor() if d.is_dynamic() else None
            sz = (s.raw_tensor.to(torch.int64) if (s is not None and s.dims) else torch.full_like(offsets, d.get_dim_value())).to(device)
            idx = torch.arange(n, device=device)[None, :] + offsets[:, None]  # [B, n]
            valid = torch.arange(n, device=device)[None, :] < sz[:, None]
            idx = torch.where(valid, idx, torch.full_like(idx, max_len))  # out-of-range -> dropped below
            out_ext_shape = list(out_shape)
            out_ext_shape[pos] = max_len + 1
            if out.shape[pos] != max_len + 1:
                out = torch.cat([out, torch.zeros_like(out.narrow(pos, 0, 1))], dim=pos)
            # move batch and pos axes to front for index_put
            o = out.movedim((bax, pos), (0, 1))
            rr = r.movedim((bax, pos), (0, 1))
            bidx = torch.arange(o.shape[0], device=device)[:, None].expand_as(idx)
            o[bidx, idx] = rr
            offsets = offsets + sz
        out = out.narrow(pos, 0, max_len)
        return wrap(out, out_dims, like=first), out_dim
    raw = torch.cat(raws, dim=pos)
    res = wrap(raw, out_dims, like=first)
    if first.feature_dim == first_dim:
        res._feature_dim = out_dim
    return res, out_dim


def concat_features(*sources: Tensor, allow_broadcast: bool = False) -> Tensor:
    """concat along each tensor's feature dim"""
    return concat(*[(s, s.feature_dim) for s in sources], allow_broadcast=allow_broadcast)[0]


def pad(source: Tensor, *, axes: Sequence[Dim], padding: Sequence[Tuple[Union[Dim, int], Union[Dim, int]]],
        out_dims: Optional[Sequence[Dim]] = None, mode: str = "constant", value=None,
        handle_dynamic_dims: Optional[bool] = None) -> Tuple[Tensor, Sequence[Dim]]:
    """
    Pad the given axes left/right. For an axis with per-sequence sizes and right padding, the padding goes directly
    after each sequence's end (``handle_dynamic_dims``), so that the result is again a valid padded batch.
    """
    assert len(axes) == len(padding)
    if handle_dynamic_dims is None:
        handle_dynamic_dims = True
    if out_dims is None:
        out_dims = []
        for a, (l, r) in zip(axes, padding):
            li = l.get_dim_value() if isinstance(l, Dim) else l
            ri = r.get_dim_value() if isinstance(r, Dim) else r
            if li == 0 and ri == 0:
                out_dims.append(a)
            else:
                out_dims.append(Dim._derive("pad", [a], attribs={"left": li, "right": ri}))
    raw = source._raw_tensor
    dims = list(source._dims)
    value_ = 0 if value is None else value
    if isinstance(value_, Tensor):
        value_ = value_._raw_tensor.item() if not value_._dims else value_
    for a, (l, r), od in zip(axes, padding, out_dims):
        li = l.get_dim_value() if isinstance(l, Dim) else l
        ri = r.get_dim_value() if isinstance(r, Dim) else r
        ax = axis_of(source, a)
        padspec = [0, 0] * (raw.ndim - ax - 1) + [li, ri]
        dyn = a.is_dynamic() and a.is_dynamic_seq_length() and ri > 0 and handle_dynamic_dims
        if mode == "constant":
            new = F.pad(raw, padspec, mode="constant", value=value_)
        else:
            m = {"reflect": "reflect", "replicate": "replicate", "circular": "circular"}[mode]
            # F.pad non-constant modes want the padded dims last and a batch dim
            new = raw.movedim(ax, -1)
            shp = new.shape
            new = F.pad(new.reshape(1, -1, shp[-1]), [li, ri], mode=m).reshape(*shp[:-1], shp[-1] + li + ri).movedim(-1, ax)
        if dyn and mode == "constant":
            # frames between seq end and the padded end hold source padding: overwrite by value
            sizes = a.get_size_tensor(device=raw.device)
            sraw = sizes.copy_compatible_to_dims_raw(dims)
            pos = torch.arange(new.shape[ax], device=raw.device).reshape([-1 if i == ax else 1 for i in range(raw.ndim)])
            in_pad = (pos >= (sraw + li)) & (pos < (sraw + li + ri))
            new = torch.where(in_pad, torch.full((), value_, dtype=new.dtype, device=new.device), new)
        raw = new
        dims[ax] = od
    res = wrap(raw, dims, like=source)
    if source.feature_dim in axes:
        res._feature_dim = out_dims[list(axes).index(source.feature_dim)]
    return res, out_dims


def cum_concat_step(source: Tensor, *, prev_accum: Tensor, axis: Dim, out_spatial_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """append one step to an accumulated sequence (incremental decoding: self-attention K/V history)"""
    if out_spatial_dim is None:
        out_spatial_dim = axis + 1
    ax = axis_of(prev_accum, axis)
    tgt_dims = list(prev_accum._dims)
    step_dims = [d for d in tgt_dims if d != axis]
    step = source.copy_compatible_to_dims_raw(step_dims).unsqueeze(ax)
    shape = list(prev_accum._raw_tensor.shape)
    shape[ax] = 1
    step = step.expand(*shape)
    raw = torch.cat([prev_accum._raw_tensor, step.to(prev_accum._raw_tensor.dtype)], dim=ax)
    tgt_dims[ax] = out_spatial_dim
    if out_spatial_dim.is_dynamic() and (out_spatial_dim.dyn_size_ext is None or out_spatial_dim.derived_from_op is None):
        out_spatial_dim.dyn_size_ext = Tensor("%s:size" % out_spatial_dim.name, dims=[], dtype="int32",
                                              raw_tensor=torch.tensor(raw.shape[ax], dtype=torch.int32))
    return wrap(raw, tgt_dims, like=prev_accum), out_spatial_dim


def stack(sources: Sequence[Tensor], *, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """stack along a new first axis (the dim order of the reference: returnn/torch/frontend/_backend.py:592)"""
    if out_dim is None:
        out_dim = Dim(len(sources), name="stack")
    dims = sources[0]._dims
    raws = [s.copy_compatible_to_dims_raw(dims) for s in sources]
    raw = torch.stack(raws, dim=0)
    return wrap(raw, [out_dim] + list(dims), like=sources[0]), out_dim


def sequence_mask(dims: Union[Dim, Sequence[Dim]], *, device: Optional[str] = None) -> Tensor:
    """bool mask over the given dims: True at valid frames of every dynamic dim"""
    if isinstance(dims, Dim):
        dims = [dims]
    mask = None
    for d in dims:
        if d.is_dynamic() and not d.is_batch_dim() and d.need_masking() and d.dyn_size_ext is not None and d.dyn_size_ext.dims:
            m = d.get_mask(device=device)
            mask = m if mask is None else (mask & m)
    if mask is None:
        return convert_to_tensor(True, device=device)
    return mask


def masked_select(tensor: Tensor, *, mask: Tensor, dims: Sequence[Dim], out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    Select the entries where mask is True, flattening ``dims`` (the mask's dims) into one new dim.
    """
    dims = list(dims)
    assert set(mask._dims) == set(dims), "masked_select: mask dims %r must equal dims %r" % (mask._dims, dims)
    rest = [d for d in tensor._dims if d not in dims]
    traw = tensor.copy_compatible_to_dims_raw(dims + rest)
    mraw = mask.copy_compatible_to_dims_raw(dims)
    if mraw.device != traw.device:
        mraw = mraw.to(traw.device)
    sel = traw[mraw]
    if out_dim is None:
        out_dim = Dim(None, name="masked_select")
    if out_dim.is_dynamic() and (out_dim.dyn_size_ext is None or out_dim.dyn_size_ext.raw_tensor is None or True):
        out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=[], dtype="int32", raw_tensor=torch.tensor(sel.shape[0], dtype=torch.int32))
    return wrap(sel, [out_dim] + rest, like=tensor), out_dim


def masked_scatter(source: Tensor, backup: Optional[Tensor] = None, *, mask: Tensor, dims: Sequence[Dim], in_dim: Dim) -> Tensor:
    """inverse of masked_select: put source[in_dim] back at the True positions; elsewhere backup (or 0)"""
    dims = list(dims)
    rest = [d for d in source._dims if d != in_dim]
    sraw = source.copy_compatible_to_dims_raw([in_dim] + rest)
    mraw = mask.copy_compatible_to_dims_raw(dims).to(sraw.device)
    shape = [d.get_dim_value() for d in dims] + list(sraw.shape[1:])
    if backup is not None:
        out = backup.copy_compatible_to_dims_raw(dims + rest).expand(*shape).clone().to(sraw.dtype)
    else:
        out = torch.zeros(shape, dtype=sraw.dtype, device=sraw.device)
    out[mraw] = sraw
    return wrap(out, dims + rest, like=source)


def pack_padded(source: Tensor, *, dims: Sequence[Dim], enforce_sorted: bool = False, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    Remove padding: flatten ``dims`` (e.g. batch and time) into one dim holding only valid frames.
    """
    mask = sequence_mask(dims, device=source.device)
    if not mask._dims:
        return merge_dims(source, dims=dims, out_dim=out_dim)
    if set(mask._dims) != set(dims):
        mask = mask.copy_compatible_to_dims(list(dims), unbroadcast=True)
    return masked_select(source, mask=mask, dims=dims, out_dim=out_dim)


def gather(source: Tensor, *, indices: Union[Tensor, int], axis: Optional[Dim] = None, clip_to_valid: bool = False) -> Tensor:
    """
    ``out[indices.dims..., rest...] = source[..., indices, ...]`` along ``axis``. Dims shared between source and indices
    act as batch dims.
    """
    if axis is None:
        assert isinstance(indices, Tensor) and indices.sparse_dim is not None
        axis = indices.sparse_dim
    ax = axis_of(source, axis)
    if isinstance(indices, int):
        dims = list(source._dims)
        dims.pop(ax)
        return wrap(source._raw_tensor.select(ax, indices), dims, like=source)
    iraw = indices._raw_tensor
    if iraw.dtype not in (torch.int64, torch.int32):
        iraw = iraw.to(torch.int64)
    if clip_to_valid:
        if axis.is_dynamic() and axis.dyn_size_ext is not None and axis.dyn_size_ext.dims:
            sizes = axis.get_size_tensor(device=iraw.device).copy_compatible_to_dims_raw(indices._dims) if all(
                d in indices._dims for d in axis.dyn_size_ext.dims) else None
            if sizes is not None:
                iraw = torch.minimum(iraw.clamp_min(0), (sizes - 1).to(iraw.dtype))
            else:
                iraw = iraw.clamp(0, source._raw_tensor.shape[ax] - 1)
        else:
            iraw = iraw.clamp(0, source._raw_tensor.shape[ax] - 1)
    common = [d for d in indices._dims if d in source._dims and d != axis]
    if not common:
        idx_flat = iraw.reshape(-1).to(source._raw_tensor.device)
        out = torch.index_select(source._raw_tensor, ax, idx_flat.to(torch.int64) if idx_flat.dtype != torch.int64 else idx_flat)
        new_shape = list(source._raw_tensor.shape[:ax]) + list(iraw.shape) + list(source._raw_tensor.shape[ax + 1:])
        out = out.reshape(new_shape)
        dims = list(source._dims[:ax]) + list(indices._dims) + list(source._dims[ax + 1:])
        res = wrap(out, dims, like=source)
        return res
    # batched gather: layout source as [common..., axis, rest...], indices as [common..., idx_rest...]
    src_rest = [d for d in source._dims if d not in common and d != axis]
    idx_rest = [d for d in indices._dims if d not in common]
    sraw = source.copy_compatible_to_dims_raw(common + [axis] + src_rest)
    iraw2 = indices.copy_with_raw(iraw).copy_compatible_to_dims_raw(common + idx_rest).to(sraw.device).to(torch.int64)
    nc = len(common)
    cshape = list(sraw.shape[:nc])
    n_axis = sraw.shape[nc]
    rest_shape = list(sraw.shape[nc + 1:])
    idx_shape = list(iraw2.shape[nc:])
    s3 = sraw.reshape([-1, n_axis] + [int(numpy.prod(rest_shape)) if rest_shape else 1])
    cshape_i = list(iraw2.shape[:nc])
    if cshape_i != cshape:
        iraw2 = iraw2.expand(*(cshape + idx_shape))
    i2 = iraw2.reshape(s3.shape[0], -1)
    out = torch.gather(s3, 1, i2.unsqueeze(-1).expand(-1, -1, s3.shape[2]))
    out = out.reshape(cshape + idx_shape + rest_shape)
    return wrap(out, common + idx_rest + src_rest, like=source)


def _scatter_impl(source: Tensor, indices: Tensor, indices_dim, out_dim, mode: str, fill_value, use_mask=True):
    if isinstance(indices_dim, Dim):
        indices_dims = [indices_dim]
    else:
        indices_dims = list(indices_dim)
    if out_dim is None:
        out_dim = indices.sparse_dim
    assert out_dim is not None
    out_dims_multi = [out_dim] if isinstance(out_dim, Dim) else list(out_dim)
    assert len(out_dims_multi) == 1, "scatter: multiple out dims: flatten the indices first"
    out_dim = out_dims_multi[0]
    common = [d for d in indices._dims if d not in indices_dims]
    src_rest = [d for d in source._dims if d not in indices_dims and d not in common]
    for d in common:
        assert d in source._dims or True
    if use_mask:
        m = sequence_mask(indices_dims, device=source.device)
    else:
        m = None
    sraw = source.copy_compatible_to_dims_raw(common + indices_dims + src_rest)
    full_shape = [d.get_dim_value() for d in common] + [d.get_dim_value() for d in indices_dims] + list(sraw.shape[len(common) + len(indices_dims):])
    sraw = sraw.expand(*full_shape)
    iraw = indices.copy_compatible_to_dims_raw(common + indices_dims).to(sraw.device).to(torch.int64)
    iraw = iraw.expand(*full_shape[: len(common) + len(indices_dims)])
    nc = len(common)
    B = int(numpy.prod(full_shape[:nc])) if nc else 1
    N = int(numpy.prod(full_shape[nc: nc + len(indices_dims)]))
    R = int(numpy.prod(full_shape[nc + len(indices_dims):])) if src_rest else 1
    s3 = sraw.reshape(B, N, R)
    i2 = iraw.reshape(B, N)
    n_out = out_dim.get_dim_value()
    if m is not None and m._dims:
        mraw = m.copy_compatible_to_dims_raw(common + indices_dims).expand(*full_shape[: nc + len(indices_dims)]).reshape(B, N).to(sraw.device)
        i2 = torch.where(mraw, i2, torch.full_like(i2, n_out))
        n_alloc = n_out + 1
    else:
        n_alloc = n_out
    idx3 = i2.unsqueeze(-1).expand(-1, -1, R)
    if mode == "sum":
        out = torch.zeros(B, n_alloc, R, dtype=s3.dtype, device=s3.device)
        out.scatter_add_(1, idx3, s3)
    elif mode in ("max", "min"):
        init = fill_value if fill_value is not None else (float("-inf") if mode == "max" else float("inf"))
        if not s3.dtype.is_floating_point and fill_value is None:
            init = torch.iinfo(s3.dtype).min if mode == "max" else torch.iinfo(s3.dtype).max
        out = torch.full((B, n_alloc, R), init, dtype=s3.dtype, device=s3.device)
        out.scatter_reduce_(1, idx3, s3, reduce="amax" if mode == "max" else "amin", include_self=True)
    elif mode == "mean":
        out = torch.zeros(B, n_alloc, R, dtype=s3.dtype, device=s3.device)
        out.scatter_reduce_(1, idx3, s3, reduce="mean", include_self=False)
    elif mode == "logsumexp":
        mx = torch.full((B, n_alloc, R), float("-inf"), dtype=s3.dtype, device=s3.device)
        mx.scatter_reduce_(1, idx3, s3, reduce="amax", include_self=True)
        mx_safe = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
        e = torch.exp(s3 - torch.gather(mx_safe, 1, idx3))
        acc = torch.zeros_like(mx)
        acc.scatter_add_(1, idx3, e)
        out = torch.log(acc) + mx_safe
        out = torch.where(acc > 0, out, torch.full_like(out, float("-inf")))
    else:
        raise ValueError("scatter: mode %r" % mode)
    if n_alloc != n_out:
        out = out[:, :n_out]
    out = out.reshape(full_shape[:nc] + [n_out] + full_shape[nc + len(indices_dims):])
    return wrap(out, common + [out_dim] + src_rest, like=source)


def scatter(source: Tensor, *, indices: Tensor, indices_dim: Union[Dim, Sequence[Dim]], mode: str = "sum",
            fill_value=None, out_dim: Optional[Union[Dim, Sequence[Dim]]] = None, use_mask: Optional[bool] = None) -> Tensor:
    """
    ``out[..., indices[i], ...] (+)= source[..., i, ...]`` for i over indices_dim. mode: sum / max / min / logsumexp / mean.
    """
    return _scatter_impl(source, indices, indices_dim, out_dim, mode, fill_value, use_mask=True if use_mask is None else use_mask)


def scatter_mean(source, *, indices, indices_dim, fill_value=None, out_dim=None) -> Tensor:
    """scatter with averaging"""
    return scatter(source, indices=indices, indices_dim=indices_dim, mode="mean", fill_value=fill_value, out_dim=out_dim)


def scatter_logsumexp(source, *, indices, indices_dim, fill_value=None, out_dim=None) -> Tensor:
    """scatter in log space"""
    return scatter(source, indices=indices, indices_dim=indices_dim, mode="logsumexp", fill_value=fill_value, out_dim=out_dim)


def scatter_logmeanexp(source, *, indices, indices_dim, fill_value=None, out_dim=None) -> Tensor:
    """log(mean(exp))"""
    ones = wrap(torch.ones_like(source._raw_tensor), source._dims)
    counts = scatter(ones, indices=indices, indices_dim=indices_dim, out_dim=out_dim)
    lse = scatter_logsumexp(source, indices=indices, indices_dim=indices_dim, out_dim=out_dim)
    from .math_ import log

    return lse - log(counts)


def scatter_argmax(source: Tensor, *, indices: Tensor, indices_dim, invalid_idx: int = -1, out_dim=None) -> Tensor:
    """for each target slot, the position in indices_dim whose source value was the max"""
    mx = scatter(source, indices=indices, indices_dim=indices_dim, mode="max", out_dim=out_dim)
    if out_dim is None:
        out_dim = indices.sparse_dim
    back = gather(mx, indices=indices, axis=out_dim)
    idim = indices_dim if isinstance(indices_dim, Dim) else indices_dim[0]
    from .dims import range_over_dim

    pos = range_over_dim(idim, device=source.device)
    is_max = source == back
    cand = where(is_max, pos, invalid_idx)
    res = scatter(cand, indices=indices, indices_dim=indices_dim, mode="max", fill_value=invalid_idx, out_dim=out_dim)
    res.sparse_dim = idim
    return res


def slice(source: Tensor, *, axis: Dim, start=None, end=None, step=None, size=None, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """``source[start:end:step]`` (or ``[start:start+size]``) along axis"""
    ax = axis_of(source, axis)
    n = source._raw_tensor.shape[ax]

    def _val(v):
        if isinstance(v, Tensor):
            assert not v._dims, "slice: per-sequence start/end: use rf.gather with a range"
            return int(v._raw_tensor)
        if isinstance(v, Dim):
            return v.get_dim_value()
        return v

    start_, end_, step_, size_ = _val(start), _val(end), _val(step), _val(size)
    if size_ is not None:
        assert end_ is None
        end_ = (start_ or 0) + size_
    import builtins

    sl = builtins.slice(start_, end_, step_)
    idx = [builtins.slice(None)] * source._raw_tensor.ndim
    idx[ax] = sl
    raw = source._raw_tensor[tuple(idx)]
    if out_dim is None:
        if axis.is_static() or not (axis.is_dynamic_seq_length()):
            if isinstance(size, Dim):
                out_dim = size
            else:
                out_dim = Dim(raw.shape[ax], name="slice") if axis.is_static() else Dim(None, name="slice")
        else:
            out_dim = Dim(None, name="slice")
    if out_dim.is_dynamic() and out_dim.derived_from_op is None:
        if axis.is_dynamic() and axis.is_dynamic_seq_length():
            sizes = axis.dyn_size_ext.raw_tensor.to(torch.int64)
            s0, e0, st = sl.indices(10**9)
            s_eff = torch.clamp(torch.where(torch.tensor(start_ is not None and start_ < 0), sizes + (start_ or 0), torch.full_like(sizes, start_ or 0)), min=0)
            if end_ is None:
                e_eff = sizes
            elif end_ < 0:
                e_eff = torch.clamp(sizes + end_, min=0)
            else:
                e_eff = torch.clamp(torch.full_like(sizes, end_), max=None).minimum(sizes)
            new_sizes = torch.clamp(-(-(e_eff - s_eff) // (step_ or 1)), min=0)
            out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=axis.dyn_size_ext.dims, dtype="int32", raw_tensor=new_sizes.to(torch.int32))
        else:
            out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=[], dtype="int32", raw_tensor=torch.tensor(raw.shape[ax], dtype=torch.int32))
    dims = list(source._dims)
    dims[ax] = out_dim
    res = wrap(raw, dims, like=source)
    if source.feature_dim == axis:
        res._feature_dim = out_dim
    return res, out_dim


def shift_right(source: Tensor, *, axis: Dim, pad_value, amount: int = 1) -> Tensor:
    """shift by amount to the right, pad left, same length (decoder input from targets)"""
    ax = axis_of(source, axis)
    raw = source._raw_tensor
    if isinstance(pad_value, Tensor):
        pad_value = pad_value._raw_tensor.item()
    padded = F.pad(raw, [0, 0] * (raw.ndim - ax - 1) + [amount, 0], value=pad_value)
    return wrap(padded.narrow(ax, 0, raw.shape[ax]), source._dims, like=source)


def shift_left(source: Tensor, *, axis: Dim, pad_value, amount: int = 1) -> Tensor:
    """shift by amount to the left, pad right"""
    ax = axis_of(source, axis)
    raw = source._raw_tensor
    if isinstance(pad_value, Tensor):
        pad_value = pad_value._raw_tensor.item()
    padded = F.pad(raw, [0, 0] * (raw.ndim - ax - 1) + [0, amount], value=pad_value)
    return wrap(padded.narrow(ax, amount, raw.shape[ax]), source._dims, like=source)


def reverse_sequence(tensor: Tensor, *, axis: Dim, handle_dynamic_dims: bool = True) -> Tensor:
    """reverse along axis; with per-sequence sizes every sequence is reversed within its own length"""
    ax = axis_of(tensor, axis)
    if not handle_dynamic_dims or not (axis.is_dynamic() and axis.is_dynamic_seq_length()):
        return wrap(torch.flip(tensor._raw_tensor, [ax]), tensor._dims, like=tensor)
    raw = tensor._raw_tensor
    sizes = axis.get_size_tensor(device=raw.device)
    T = raw.shape[ax]
    ext_dims = list(sizes._dims) + [axis]
    pos = torch.arange(T, device=raw.device)
    s = sizes._raw_tensor.to(torch.int64).unsqueeze(-1)
    idx = torch.where(pos < s, s - 1 - pos, pos.expand(*s.shape[:-1], T))
    idx_t = wrap(idx, ext_dims)
    return gather(tensor, indices=idx_t, axis=axis).copy_transpose_to_dims(tensor._dims)


def where(cond: Union[Tensor, bool], true_: Union[Tensor, int, float, bool], false_: Union[Tensor, int, float, bool],
          *, allow_broadcast_all_sources: bool = False) -> Tensor:
    """element-wise select"""
    if isinstance(cond, bool):
        res = true_ if cond else false_
        return res if isinstance(res, Tensor) else _convert_to_tensor(res)
    like = true_ if isinstance(true_, Tensor) else (false_ if isinstance(false_, Tensor) else None)
    t = true_ if isinstance(true_, Tensor) else _convert_to_tensor(true_, like=like, device=cond.device)
    f = false_ if isinstance(false_, Tensor) else _convert_to_tensor(false_, like=like if like is not None else t, device=cond.device)
    cands = sorted([cond, t, f], key=lambda x: -len(x._dims))
    out_dims = list(cands[0]._dims)
    for c in cands[1:]:
        for d in c._dims:
            if d not in out_dims:
                out_dims.append(d)
    # keep the order of the value tensor with most dims if it covers everything
    for c in (t, f):
        if set(c._dims) == set(out_dims):
            out_dims = list(c._dims)
            break
    craw = cond.copy_compatible_to_dims_raw(out_dims)
    traw = t.copy_compatible_to_dims_raw(out_dims) if t._dims else t._raw_tensor
    fraw = f.copy_compatible_to_dims_raw(out_dims) if f._dims else f._raw_tensor
    dev = traw.device if traw.ndim else (fraw.device if fraw.ndim else craw.device)
    if craw.device != dev:
        craw = craw.to(dev)
    if traw.device != dev:
        traw = traw.to(dev)
    if fraw.device != dev:
        fraw = fraw.to(dev)
    if traw.dtype != fraw.dtype:
        if not t._dims:
            traw = traw.to(fraw.dtype)
        else:
            fraw = fraw.to(traw.dtype)
    return wrap(torch.where(craw, traw, fraw), out_dims, like=t if t._dims else f)


def search_sorted(sorted_seq: Tensor, values: Tensor, *, axis: Dim, side: str = "left", out_dtype: str = "int32") -> Tensor:
    """positions where values would be inserted into sorted_seq along axis"""
    rest = [d for d in sorted_seq._dims if d != axis]
    vrest = [d for d in values._dims if d not in rest]
    sraw = sorted_seq.copy_compatible_to_dims_raw(rest + [axis])
    vraw = values.copy_compatible_to_dims_raw(rest + vrest)
    vshape = list(vraw.shape)
    vflat = vraw.reshape(list(sraw.shape[:-1]) + [-1]) if rest else vraw.reshape(-1)
    if rest:
        vflat = vraw.expand(*[s if s != 1 else ss for s, ss in zip(vraw.shape[: len(rest)], sraw.shape[:-1])], *vraw.shape[len(rest):]).reshape(list(sraw.shape[:-1]) + [-1])
    res = torch.searchsorted(sraw.contiguous(), vflat.contiguous(), right=(side == "right"))
    res = res.reshape(list(sraw.shape[:-1]) + vshape[len(rest):]).to(torch_dtype(out_dtype))
    return wrap(res, rest + vrest, sparse_dim=axis)


def sparse_to_dense(labels: Union[Tensor, int], *, label_value=1.0, other_value=0.0, axis: Optional[Dim] = None) -> Tensor:
    """one-hot with custom on/off values; the class axis goes last"""
    if axis is None:
        axis = labels.sparse_dim
    assert axis is not None
    raw = labels._raw_tensor.to(torch.int64)
    oh = F.one_hot(raw, axis.get_dim_value()).to(torch.bool)
    on = label_value._raw_tensor if isinstance(label_value, Tensor) else torch.tensor(label_value, device=raw.device)
    off = other_value._raw_tensor if isinstance(other_value, Tensor) else torch.tensor(other_value, device=raw.device)
    if not on.dtype.is_floating_point and isinstance(label_value, float):
        on = on.float()
    out = torch.where(oh, on.to(raw.device), off.to(raw.device).to(on.dtype))
    return wrap(out, list(labels._dims) + [axis], feature_dim=axis)


def one_hot(source: Tensor) -> Tensor:
    """float one-hot over source.sparse_dim"""
    return sparse_to_dense(source, label_value=1.0, other_value=0.0)


def sort(source: Tensor, *, axis: Dim, descending: bool = False, stable: bool = True) -> Tuple[Tensor, Tensor, Dim]:
    """:return: sorted values, indices (sparse over axis), out dim (a copy of axis)"""
    ax = axis_of(source, axis)
    vals, idx = torch.sort(source._raw_tensor, dim=ax, descending=descending, stable=stable)
    out_dim = axis.copy(same_as_self=False, description="%s:sorted" % axis.name)
    dims = list(source._dims)
    dims[ax] = out_dim
    return wrap(vals, dims, like=source), wrap(idx.to(torch.int32), dims, sparse_dim=axis), out_dim


def top_k_mask(values: Tensor, *, axis: Dim, k: Union[int, Tensor]) -> Tensor:
    """True for the k largest entries along axis"""
    ax = axis_of(values, axis)
    kk = int(k._raw_tensor) if isinstance(k, Tensor) else k
    kth = torch.topk(values._raw_tensor, kk, dim=ax).values.narrow(ax, kk - 1, 1)
    return wrap(values._raw_tensor >= kth, values._dims)


def top_p_mask(probs: Tensor, *, p: Union[float, Tensor], axis: Dim, one_more: bool = True) -> Tensor:
    """nucleus: True for the smallest set of entries whose probability mass reaches p"""
    ax = axis_of(probs, axis)
    raw = probs._raw_tensor
    sorted_p, idx = torch.sort(raw, dim=ax, descending=True)
    cum = torch.cumsum(sorted_p, dim=ax)
    praw = p._raw_tensor if isinstance(p, Tensor) else p
    m = cum <= praw
    if one_more:
        m = torch.cat([torch.ones_like(m.narrow(ax, 0, 1)), m.narrow(ax, 0, m.shape[ax] - 1)], dim=ax)
    out = torch.zeros_like(m)
    out.scatter_(ax, idx, m)
    return wrap(out, probs._dims)


def repeat(values: Tensor, *, in_spatial_dim: Dim, repeats: Union[int, Tensor], out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """repeat each frame ``repeats`` times (int: uniform; Tensor [.., in_spatial_dim]: per frame durations)"""
    ax = axis_of(values, in_spatial_dim)
    if isinstance(repeats, int):
        raw = torch.repeat_interleave(values._raw_tensor, repeats, dim=ax)
        if out_dim is None:
            out_dim = in_spatial_dim * repeats
        dims = list(values._dims)
        dims[ax] = out_dim
        return wrap(raw, dims, like=values), out_dim
    # per-frame durations -> gather indices via searchsorted on cumsum
    rep = repeats.copy_masked(0)
    rraw = rep.copy_compatible_to_dims_raw([d for d in rep._dims if d != in_spatial_dim] + [in_spatial_dim]).to(torch.int64)
    cum = torch.cumsum(rraw, dim=-1)
    total = cum[..., -1]
    max_len = int(total.max()) if total.numel() else 0
    pos = torch.arange(max_len, device=rraw.device)
    idx = torch.searchsorted(cum, pos.expand(*cum.shape[:-1], max_len).contiguous(), right=True)
    idx = idx.clamp(max=rraw.shape[-1] - 1)
    if out_dim is None:
        out_dim = Dim(None, name="repeat")
    bd = [d for d in rep._dims if d != in_spatial_dim]
    out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=bd, dtype="int32", raw_tensor=total.to(torch.int32).cpu())
    res = gather(values, indices=wrap(idx, bd + [out_dim], sparse_dim=in_spatial_dim), axis=in_spatial_dim)
    return res, out_dim


def tile(source: Tensor, *, axis: Dim, multiples: int, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """concatenate multiples copies along axis"""
    ax = axis_of(source, axis)
    reps = [1] * source._raw_tensor.ndim
    reps[ax] = multiples
    if out_dim is None:
        out_dim = multiples * axis
    dims = list(source._dims)
    dims[ax] = out_dim
    return wrap(source._raw_tensor.repeat(*reps), dims, like=source), out_dim


def cumsum(source: Tensor, *, spatial_dim: Dim) -> Tensor:
    """cumulative sum along spatial_dim"""
    ax = axis_of(source, spatial_dim)
    return wrap(torch.cumsum(source._raw_tensor, dim=ax, dtype=source._raw_tensor.dtype), source._dims, like=source)


def nonzero_indices(mask: Tensor, *, out_dim: Optional[Dim] = None):
    """indices of True entries of a 1-D mask"""
    assert len(mask._dims) == 1
    idx = torch.nonzero(mask._raw_tensor, as_tuple=False).squeeze(-1).to(torch.int32)
    if out_dim is None:
        out_dim = Dim(None, name="nonzero")
    out_dim.dyn_size_ext = Tensor("%s:size" % out_dim.name, dims=[], dtype="int32", raw_tensor=torch.tensor(idx.shape[0], dtype=torch.int32))
    return wrap(idx, [out_dim], sparse_dim=mask._dims[0]), out_dim


def unstack(source: Tensor, *, axis: Dim) -> Tuple[Tensor, ...]:
    """
    ``axis.dimension`` tensors, each ``source`` without ``axis`` (views, nothing is copied): the inverse of :func:`stack`.
    Reference: returnn/frontend/array_.py:662-677.
    """
    if axis.dimension is None:
        raise ValueError("unstack: axis %s must be static (known dimension)" % (axis,))
    ax = source.get_axis_from_description(axis)
    rest = [d for i, d in enumerate(source.dims) if i != ax]
    return tuple(wrap(raw, rest, like=source, name="unstack") for raw in torch.unbind(source.raw_tensor, dim=ax))


def scatter_count(*, indices: Tensor, indices_dim: Union[Dim, Sequence[Dim]], out_dim: Optional[Union[Dim, Sequence[Dim]]] = None,
                  fill_value: Optional[int] = None) -> Tensor:
    """
    How often every index occurs in ``indices`` (int32 counts over ``out_dim``, default: the sparse dim of the indices); entries
    that never occur get ``fill_value`` (default 0).  Reference: returnn/frontend/array_.py:997-1022.
    """
    from .const import ones

    counts = scatter(ones(dims=indices.dims, dtype="int32", device=indices.device), indices=indices, indices_dim=indices_dim, out_dim=out_dim)
    if fill_value:
        counts = where(counts > 0, counts, fill_value)
    return counts


def pad_packed(source: Tensor, *, in_dim: Dim, dims: Sequence[Dim]) -> Tensor:
    """inverse of :func:`pack_padded`: the packed axis ``in_dim`` back to the padded ``dims`` (zeros behind the sequence ends)"""
    mask = sequence_mask(dims, device=source.device)
    return masked_scatter(source, mask=mask, in_dim=in_dim, dims=dims)


def expand_make_non_empty(source: Tensor, *, axis: Dim, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    ``axis`` made at least one entry long: unchanged if it is not empty, else one zero entry (some kernels cannot take empty
    tensors).  Reference: returnn/frontend/array_.py:1537-1561.
    """
    ax = source.get_axis_from_description(axis)
    if source.raw_tensor.shape[ax] > 0:
        return source, axis
    padded, (new_axis,) = pad(source, axes=[axis], padding=[(0, 1)], mode="constant", value=0)
    if out_dim is not None:
        from .dims import replace_dim

        padded, new_axis = replace_dim(padded, in_dim=new_axis, out_dim=out_dim)
    return padded, new_axis


def real_as_complex(x: Tensor, *, pair_dim: Dim) -> Tensor:
    """
    A real tensor whose size-2 ``pair_dim`` holds (real, imaginary) -> complex tensor without that dim (float32 -> complex64,
    float64 -> complex128).  Reference: returnn/frontend/array_.py:1564-1589.
    """
    if pair_dim.dimension != 2:
        raise ValueError("real_as_complex: pair_dim %s must have size 2" % (pair_dim,))
    ax = x.get_axis_from_description(pair_dim)
    raw = x.raw_tensor.movedim(ax, -1).contiguous()
    rest = [d for i, d in enumerate(x.dims) if i != ax]
    out = torch.view_as_complex(raw)
    return wrap(out, rest, name="real_as_complex")


def complex_as_real(x: Tensor, *, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """complex tensor -> real tensor with a new last dim of size 2 (real, imaginary); returns the tensor and that dim"""
    if out_dim is None:
        out_dim = Dim(2, name="complex")
    assert out_dim.dimension == 2
    return wrap(torch.view_as_real(x.raw_tensor), list(x.dims) + [out_dim], name="complex_as_real"), out_dim


def make_complex(real: Tensor, imag: Tensor) -> Tensor:
    """complex tensor from its parts (dims: union of the operands' dims)"""
    from .math_ import _prep_bin

    a, b, ra, rb, out_dims = _prep_bin(real, imag, None, None)
    ra, rb = torch.broadcast_tensors(ra, rb)
    if ra.dtype != rb.dtype:
        rb = rb.to(ra.dtype)
    return wrap(torch.complex(ra.contiguous(), rb.contiguous()), out_dims, name="make_complex")
