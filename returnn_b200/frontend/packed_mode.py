"""
Packed execution of ordinary RF models: between ``pack_padded_tensor`` and ``unpack_to_padded`` a ``[batch, time, ...]`` tensor
travels as ``[rows, ...]`` with only the valid frames of all sequences back to back, as a normal :class:`Tensor` whose first dim
is a *packed dim* (a dynamic :class:`Dim` that remembers which (batch, time) dims it stands for and the sequence offsets).

Row-wise modules (Linear, LayerNorm, activations, dropout, residual sums, BatchNorm statistics) need no change: they see a
2-D tensor without padding. Modules that work along time are called, as always, with the original time dim
(``spatial_dim=time`` / ``axis=time``); they find that their input does not have that dim but a packed dim standing for it
(:func:`packed_dim_of`) and run their packed form:

* ``RelPosSelfAttention`` / ``SelfAttention``: the varlen attention kernels on the packed qkv rows (``ops/attention_packed.py``);
* convolution / pooling along time, and anything else without a packed kernel: :func:`apply_padded` unpacks, applies the padded
  op and packs the result (also when the op changes the time dim, e.g. by striding: the result gets a new packed dim).

``ConformerEncoder`` packs behind its (2-D convolutional) frontend and unpacks at its output when packed mode is on: config key
``packed_tensors`` (``True`` or a dict) or the context manager :func:`packed_mode_ctx`.

Reference: the packed raw-tensor type and its op table in returnn/frontend/_packed_backend.py:186 (PackedRawTensor), :4238
(pack / unpack); here the sequence structure rides on the Dim instead of on a second raw-tensor class.
"""

from __future__ import annotations
from typing import Callable, Optional, Sequence, Tuple
import contextlib
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap

__all__ = ["PackedDimInfo", "pack_padded_tensor", "unpack_to_padded", "packed_dim_of", "apply_padded", "is_enabled", "packed_mode_ctx"]

_override: Optional[bool] = None


def is_enabled() -> bool:
    """packed mode requested: :func:`packed_mode_ctx`, else the global config's ``packed_tensors``"""
    if _override is not None:
        return _override
    from ..config import get_global_config

    cfg = get_global_config(raise_exception=False)
    return bool(cfg and cfg.typed_value("packed_tensors", None))


@contextlib.contextmanager
def packed_mode_ctx(enabled: bool = True):
    """force packed mode on / off inside the block"""
    global _override
    old, _override = _override, enabled
    try:
        yield
    finally:
        _override = old


class PackedDimInfo:
    """what a packed dim stands for: ``batch_dims = (batch, time)`` and the layout of the rows (a ``models.packing.PackInfo``)"""

    def __init__(self, batch_dim: Dim, time_dim: Dim, pack):
        self.batch_dim = batch_dim
        self.time_dim = time_dim
        self.pack = pack

    @property
    def batch_dims(self) -> Tuple[Dim, Dim]:
        """(batch, time)"""
        return self.batch_dim, self.time_dim


def _info(d: Dim) -> Optional[PackedDimInfo]:
    return getattr(d, "packed_info", None)


def packed_dim_of(x: Tensor, axis: Dim) -> Optional[Dim]:
    """the packed dim of ``x`` that stands for ``axis`` (None: ``x`` has ``axis`` itself, or nothing packed over it)"""
    if axis in x.dims:
        return None
    for d in x.dims:
        info = _info(d)
        if info is not None and (axis == info.time_dim or axis == info.batch_dim):
            return d
    return None


def pack_padded_tensor(x: Tensor, *, dims: Sequence[Dim], like: Optional[Dim] = None) -> Tensor:
    """
    ``[batch, time, ...] -> [rows, ...]``. ``like``: an existing packed dim over the same (batch, time): its layout is reused
    (no new index tensors, and tensors packed this way can be added to each other).
    """
    from ..models.packing import PackInfo

    bdim, tdim = dims
    if like is not None:
        info = _info(like)
        assert info is not None and info.batch_dims == (bdim, tdim)
        pdim = like
    else:
        if tdim.dyn_size_ext is not None and tdim.dyn_size_ext.dims:
            lens = tdim.dyn_size_ext.copy_compatible_to_dims_raw([bdim]).to(torch.int32).cpu()
        else:
            lens = torch.full([bdim.get_dim_value()], tdim.get_dim_value(), dtype=torch.int32)
        info = PackedDimInfo(bdim, tdim, PackInfo(lens, x.raw_tensor.device, padded_len=int(x.raw_tensor.shape[x.dims.index(tdim)])))
        pdim = Dim(None, name="packed(%s,%s)" % (bdim.name, tdim.name))
        pdim.dyn_size_ext = Tensor("%s:size" % pdim.name, dims=[], dtype="int32", raw_tensor=torch.tensor(info.pack.n, dtype=torch.int32))
        pdim.packed_info = info
    rest = [d for d in x.dims if d not in (bdim, tdim)]
    raw = x.copy_compatible_to_dims_raw([bdim, tdim] + rest)
    info = _info(pdim)
    if raw.shape[1] != info.pack.padded_len:  # same sequences, other padding (a batch-dependent maximum)
        assert raw.shape[1] >= info.pack.max_len
        raw = raw[:, : info.pack.padded_len] if raw.shape[1] > info.pack.padded_len else torch.nn.functional.pad(
            raw, [0, 0] * (raw.dim() - 2) + [0, info.pack.padded_len - raw.shape[1]])
    return wrap(info.pack.pack(raw.contiguous()), [pdim] + rest, like=x)


def unpack_to_padded(x: Tensor, pdim: Optional[Dim] = None, *, pad_value=0) -> Tensor:
    """``[rows, ...] -> [batch, time, ...]`` (time as long as the longest sequence of the batch)"""
    if pdim is None:
        pdim = next(d for d in x.dims if _info(d) is not None)
    info = _info(pdim)
    rest = [d for d in x.dims if d != pdim]
    raw = x.copy_compatible_to_dims_raw([pdim] + rest)
    pack = info.pack
    out = raw.new_full((pack.batch * pack.max_len,) + tuple(raw.shape[1:]), pad_value)
    idx = pack.row_batch.long() * pack.max_len + pack.row_pos.long()
    out.index_copy_(0, idx, raw)
    out = out.reshape((pack.batch, pack.max_len) + tuple(raw.shape[1:]))
    return wrap(out, [info.batch_dim, info.time_dim] + rest, like=x)


def apply_padded(fn: Callable[[Tensor], object], x: Tensor, pdim: Dim):
    """
    ``fn`` on the padded form of ``x``; tensors in the result that still have (batch, some time dim) are packed again: over the same
    packed dim when the time dim is unchanged, over a new one otherwise. ``fn`` may return a Tensor or a tuple whose first
    entry is the Tensor and whose further entries (e.g. new spatial dims) are passed through.
    """
    info = _info(pdim)
    res = fn(unpack_to_padded(x, pdim))
    rest_out = ()
    if isinstance(res, tuple):
        res, rest_out = res[0], res[1:]
    if info.batch_dim in res.dims:
        if info.time_dim in res.dims:
            res = pack_padded_tensor(res, dims=info.batch_dims, like=pdim)
        else:
            new_time = [d for d in res.dims if d.is_dynamic() and d.dyn_size_ext is not None and d.dyn_size_ext.dims and info.batch_dim in d.dyn_size_ext.dims]
            if len(new_time) == 1:
                res = pack_padded_tensor(res, dims=(info.batch_dim, new_time[0]))
    return (res,) + tuple(rest_out) if rest_out else res
