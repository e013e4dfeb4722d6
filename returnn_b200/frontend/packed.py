"""
Packed (ragged) tensors: ``[sum(len), F]`` storage plus ``seq_starts`` / ``seq_lens``, no padding.

``rf.pack`` converts a padded ``[B, T, ...]`` tensor into a :class:`PackedTensor`; row-wise ops (linear, norms,
activations, dropout) apply to the packed rows directly; sequence ops (self-attention, depthwise conv, CTC) take the
offsets. The flagship models run in this layout end to end (:mod:`returnn_b200.models`), with a fixed row capacity
so that one CUDA graph serves every batch.

Parity: returnn/frontend/_packed_backend.py (PackedRawTensor :186, pack/unpack :4238, pack_import),
returnn/datasets/packing.py.
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple
import torch
from ..tensor import Tensor, Dim, batch_dim
from ._utils import wrap

__all__ = ["PackedTensor", "pack", "unpack", "pack_import", "is_packed", "packed_regap", "packed_flat_content"]


class PackedTensor:
    """
    Rows of all sequences back to back.

    :ivar data: Tensor [packed_dim, ...feature dims]
    :ivar packed_dim: Dim over rows (dynamic scalar size = total valid rows; ``capacity`` = allocated rows)
    :ivar batch_dims: the dims that were packed, e.g. (batch_dim, time_dim)
    :ivar seq_starts: int32 [B] first row of each sequence (device)
    :ivar seq_lens: int32 [B] (device)
    :ivar seq_lens_host: int32 [B] host copy
    """

    def __init__(self, data: Tensor, *, packed_dim: Dim, batch_dims: Sequence[Dim], seq_starts: torch.Tensor,
                 seq_lens: torch.Tensor, seq_lens_host: Optional[torch.Tensor] = None, max_len: Optional[int] = None, gap: int = 0, align: int = 1):
        self.data = data
        self.gap, self.align = int(gap), int(align)  # empty rows after every sequence; sequence starts are multiples of ``align``
        self.packed_dim = packed_dim
        self.batch_dims = tuple(batch_dims)
        self.seq_starts = seq_starts
        self.seq_lens = seq_lens
        self.seq_lens_host = seq_lens_host if seq_lens_host is not None else seq_lens.cpu()
        self.max_len = int(self.seq_lens_host.max()) if max_len is None and self.seq_lens_host.numel() else (max_len or 0)

    @property
    def raw_tensor(self) -> torch.Tensor:
        """[rows, ...]"""
        return self.data.raw_tensor

    @property
    def num_seqs(self) -> int:
        """B"""
        return int(self.seq_lens_host.shape[0])

    @property
    def num_rows(self) -> int:
        """valid rows"""
        return int(self.seq_lens_host.sum())

    def with_data(self, data: Tensor) -> "PackedTensor":
        """same layout, other row data (result of a row-wise op)"""
        assert data.dims[0] == self.packed_dim
        return PackedTensor(data, packed_dim=self.packed_dim, batch_dims=self.batch_dims, seq_starts=self.seq_starts,
                            seq_lens=self.seq_lens, seq_lens_host=self.seq_lens_host, max_len=self.max_len, gap=self.gap, align=self.align)

    def map_rows(self, fn) -> "PackedTensor":
        """apply a row-wise RF function"""
        return self.with_data(fn(self.data))

    def __repr__(self):
        return "PackedTensor{%r, seqs=%i, rows=%i}" % (self.data, self.num_seqs, self.num_rows)


def is_packed(x) -> bool:
    """whether x is a PackedTensor"""
    return isinstance(x, PackedTensor)


def pack(x: Tensor, *, dims: Sequence[Dim], out_dim: Optional[Dim] = None, capacity: Optional[int] = None) -> PackedTensor:
    """
    :param x: padded tensor with dims (batch, time, ...)
    :param dims: (batch_dim, time_dim)
    :param capacity: allocate this many rows (zero filled past the valid ones)
    """
    bdim, tdim = dims
    rest = [d for d in x.dims if d not in dims]
    raw = x.copy_compatible_to_dims_raw([bdim, tdim] + rest)
    B, T = raw.shape[0], raw.shape[1]
    if tdim.is_dynamic() and tdim.dyn_size_ext is not None and tdim.dyn_size_ext.dims:
        lens_host = tdim.dyn_size_ext.raw_tensor.to(torch.int32).cpu()
    else:
        lens_host = torch.full([B], T, dtype=torch.int32)
    lens = lens_host.to(raw.device)
    starts_host = torch.cumsum(lens_host, 0, dtype=torch.int32) - lens_host
    mask = torch.arange(T, device=raw.device)[None, :] < lens[:, None]
    rows = raw[mask]
    n = rows.shape[0]
    if capacity is not None and capacity > n:
        rows = torch.cat([rows, rows.new_zeros(capacity - n, *rows.shape[1:])], dim=0)
    if out_dim is None:
        out_dim = Dim(None, name="packed", capacity=capacity)
    out_dim.dyn_size_ext = Tensor("packed:size", dims=[], dtype="int32", raw_tensor=torch.tensor(rows.shape[0], dtype=torch.int32))
    data = wrap(rows, [out_dim] + rest, like=x)
    return PackedTensor(data, packed_dim=out_dim, batch_dims=(bdim, tdim), seq_starts=starts_host.to(raw.device),
                        seq_lens=lens, seq_lens_host=lens_host)


def unpack(p: PackedTensor, *, pad_value=0) -> Tensor:
    """back to padded [B, T, ...]"""
    if p.gap != 0 or p.align != 1:
        p = packed_regap(p, 0, align=1)
    bdim, tdim = p.batch_dims
    raw = p.raw_tensor
    B, T = p.num_seqs, p.max_len
    out = raw.new_full((B, T) + tuple(raw.shape[1:]), pad_value)
    mask = torch.arange(T, device=raw.device)[None, :] < p.seq_lens[:, None]
    out[mask] = raw[: p.num_rows]
    return wrap(out, [bdim, tdim] + list(p.data.dims[1:]), like=p.data)


def pack_import(rows: torch.Tensor, seq_lens: torch.Tensor, *, batch_dims: Sequence[Dim], feature_dims: Sequence[Dim] = (),
                sparse_dim: Optional[Dim] = None, capacity: Optional[int] = None) -> PackedTensor:
    """wrap rows that are already packed (collate in packed mode, ``packed_tensors`` config)"""
    lens_host = seq_lens.to(torch.int32).cpu()
    starts_host = torch.cumsum(lens_host, 0, dtype=torch.int32) - lens_host
    out_dim = Dim(None, name="packed", capacity=capacity)
    out_dim.dyn_size_ext = Tensor("packed:size", dims=[], dtype="int32", raw_tensor=torch.tensor(rows.shape[0], dtype=torch.int32))
    data = wrap(rows, [out_dim] + list(feature_dims), sparse_dim=sparse_dim)
    return PackedTensor(data, packed_dim=out_dim, batch_dims=batch_dims, seq_starts=starts_host.to(rows.device),
                        seq_lens=lens_host.to(rows.device), seq_lens_host=lens_host)


def _layout_starts(lens_host: torch.Tensor, gap: int, align: int) -> Tuple[torch.Tensor, int]:
    """first row of every sequence and the total number of rows for sequences laid out with ``gap`` empty rows after each, starts aligned"""
    starts, pos = [], 0
    for n in lens_host.tolist():
        pos = -(-pos // align) * align
        starts.append(pos)
        pos += int(n) + gap
    return torch.tensor(starts, dtype=torch.int32), pos


def packed_regap(source: PackedTensor, gap: int, *, align: Optional[int] = None, total_bound: Optional[int] = None) -> PackedTensor:
    """
    The same sequences in another packed layout: ``gap`` rows of zeros after every sequence (a convolution or a window over the packed
    rows then sees zeros, not the neighbouring sequence, within ``gap`` rows of a boundary) and every sequence starting at a multiple of
    ``align`` rows (tile-aligned starts for kernels). One gather over the rows, no padded intermediate.

    :param total_bound: allocate exactly this many rows (a static buffer size; must hold the layout)
    :return: packed tensor with the new layout (``source`` itself if it already has it)
    Parity: returnn/frontend/_packed_backend.py:4363.
    """
    align = source.align if align is None else int(align)
    assert gap >= 0 and align >= 1
    if source.gap == gap and source.align == align and (total_bound is None or source.raw_tensor.shape[0] == total_bound):
        return source
    lens_host = source.seq_lens_host
    new_starts, total = _layout_starts(lens_host, gap, align)
    rows_out = total if total_bound is None else int(total_bound)
    assert rows_out >= total, "packed_regap: total_bound %i is smaller than the layout (%i rows)" % (rows_out, total)
    raw = source.raw_tensor
    dev = raw.device
    # row r of the output belongs to sequence seg[r] (or to no sequence: gaps, alignment holes, the tail)
    old_starts = source.seq_starts.to(torch.int64)
    ns = new_starts.to(dev).to(torch.int64)
    lens = source.seq_lens.to(torch.int64)
    r = torch.arange(rows_out, device=dev, dtype=torch.int64)
    seg = torch.clamp(torch.searchsorted(ns, r, right=True) - 1, min=0)
    off = r - ns[seg]
    valid = off < lens[seg]
    src_row = torch.where(valid, old_starts[seg] + off, torch.zeros_like(off))
    out = raw.index_select(0, src_row)
    out = torch.where(valid.reshape(-1, *([1] * (out.dim() - 1))), out, torch.zeros((), dtype=out.dtype, device=dev))
    out_dim = Dim(None, name="packed_regap", capacity=rows_out if total_bound is not None else None)
    out_dim.dyn_size_ext = Tensor("packed:size", dims=[], dtype="int32", raw_tensor=torch.tensor(rows_out, dtype=torch.int32))
    data = wrap(out, [out_dim] + list(source.data.dims[1:]), like=source.data)
    return PackedTensor(data, packed_dim=out_dim, batch_dims=source.batch_dims, seq_starts=new_starts.to(dev), seq_lens=source.seq_lens,
                        seq_lens_host=lens_host, max_len=source.max_len, gap=gap, align=align)


def packed_flat_content(source: PackedTensor, *, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    The content as a plain tensor over ONE flat dim in the dense layout (no gaps): what ``rf.pack_padded`` over (batch, time) gives for the
    padded form, without going through it. Rows beyond the content (a capacity tail) are zero.

    :return: (tensor ``[flat, ...]``, the flat dim; its size is the number of valid rows)
    Parity: returnn/frontend/_packed_backend.py:4151.
    """
    p = packed_regap(source, 0, align=1) if (source.gap != 0 or source.align != 1) else source
    n = p.num_rows
    raw = p.raw_tensor
    if raw.shape[0] > n:
        raw = torch.cat([raw[:n], torch.zeros_like(raw[n:])], dim=0)
    if out_dim is None:
        out_dim = Dim(None, name="packed_flat", capacity=p.packed_dim.capacity)
    if out_dim.dyn_size_ext is None or out_dim.dyn_size_ext.raw_tensor is None:
        out_dim.dyn_size_ext = Tensor("packed_flat:size", dims=[], dtype="int32", raw_tensor=torch.tensor(n, dtype=torch.int32))
    if out_dim.capacity is None and raw.shape[0] > n:
        raw = raw[:n]
    return wrap(raw, [out_dim] + list(p.data.dims[1:]), like=p.data), out_dim
