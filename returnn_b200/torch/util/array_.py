"""
Tensor helpers without data-dependent host synchronisation: masked selection with a static output size, ``nonzero`` with a
known count, sequence masks.

Parity: returnn/torch/util/array_.py (masked_select_bound :11, masked_select :127, nonzero :159, sequence_mask :181,
sequence_mask_time_major :196).
"""

from __future__ import annotations
from typing import Optional, Tuple, Union
import torch


def _flatten_for_mask(x: torch.Tensor, mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.ndim >= mask.ndim and tuple(x.shape[: mask.ndim]) == tuple(mask.shape), "mask dims must be the leading dims of the input"
    return x.reshape((-1,) + tuple(x.shape[mask.ndim:])), mask.reshape(-1)


class _PackRows(torch.autograd.Function):
    """out[s] = x[src[s]] for valid slots, else 0; the backward is a gather too (dx[r] = dout[dst[r]] for selected rows)"""

    @staticmethod
    def forward(ctx, x, src, dst, valid, selected):
        ctx.save_for_backward(dst, selected)
        out = x.index_select(0, src)
        return out * valid.reshape((-1,) + (1,) * (x.ndim - 1)).to(out.dtype)

    @staticmethod
    def backward(ctx, dout):
        dst, selected = ctx.saved_tensors
        pad = torch.zeros((1,) + tuple(dout.shape[1:]), dtype=dout.dtype, device=dout.device)
        dx = torch.cat([dout, pad], 0).index_select(0, dst)
        dx = dx * selected.reshape((-1,) + (1,) * (dout.ndim - 1)).to(dx.dtype)
        return dx, None, None, None, None


def masked_select_bound(input: torch.Tensor, mask: torch.Tensor, *, bound: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    Selected rows packed at the front of a buffer of ``bound`` rows (zeros behind), in input order. Static output shape and
    no host synchronisation: usable inside a captured CUDA graph.

    :param input: [mask_dims..., rest...]
    :param mask: [mask_dims...] bool
    :param bound: promised upper bound of the number of selected rows (default: all rows). Rows beyond it are dropped.
    :return: (out [bound, rest...], number of selected rows as an int64 scalar on the device)
    """
    x, m = _flatten_for_mask(input, mask)
    n = m.shape[0]
    if bound is None:
        bound = n
    rank = torch.cumsum(m.to(torch.int64), 0) - 1  # position among the selected rows
    count = m.sum()
    keep = m & (rank < bound)
    dst = torch.where(keep, rank, torch.full_like(rank, bound))  # slot of every input row; `bound` = dump slot
    src = torch.zeros(bound + 1, dtype=torch.int64, device=x.device)
    src.scatter_(0, dst, torch.arange(n, dtype=torch.int64, device=x.device))  # a 1-D int scatter only
    valid = torch.arange(bound, dtype=torch.int64, device=x.device) < count
    out = _PackRows.apply(x, src[:bound], dst, valid, keep)
    return out, count


def masked_select(input: torch.Tensor, mask: torch.Tensor, *, mask_len: Optional[Union[int, torch.Tensor]] = None):
    """
    ``input[mask]`` over the leading dims, via one ``nonzero`` on the flat mask and an index_select (no broadcast of the mask
    to the full input shape, which is what makes :func:`torch.masked_select` slow and memory hungry).

    :param mask_len: number of True entries if known (checked)
    :return: [mask_len, rest...]
    """
    x, m = _flatten_for_mask(input, mask)
    idx = torch.nonzero(m).squeeze(1)
    if mask_len is not None:
        assert idx.shape[0] == int(mask_len)
    return x.index_select(0, idx)


def nonzero(mask: torch.Tensor, *, out_len: Union[int, torch.Tensor]) -> torch.Tensor:
    """indices of the True entries of a flat bool mask when their number is known: a stable sort, no synchronisation"""
    assert mask.ndim == 1 and mask.dtype == torch.bool
    order = torch.sort(mask.to(torch.int8), stable=True, descending=True).indices
    return order[: int(out_len) if not isinstance(out_len, torch.Tensor) else out_len]


def sequence_mask(lengths: torch.Tensor, *, maxlen: Optional[int] = None) -> torch.Tensor:
    """[batch..., maxlen] bool, True inside the sequences"""
    if maxlen is None:
        maxlen = int(lengths.max())
    pos = torch.arange(maxlen, dtype=lengths.dtype, device=lengths.device)
    return pos < lengths.unsqueeze(-1)


def sequence_mask_time_major(lengths: torch.Tensor, *, maxlen: Optional[int] = None) -> torch.Tensor:
    """[maxlen, batch...] bool"""
    if maxlen is None:
        maxlen = int(lengths.max())
    pos = torch.arange(maxlen, dtype=lengths.dtype, device=lengths.device)
    return pos.reshape((-1,) + (1,) * lengths.ndim) < lengths.unsqueeze(0)
