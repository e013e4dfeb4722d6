"""
Packed-row layout helpers for the fused model paths: valid frames of all sequences back to back in ``[N, F]``,
``cu_seqlens`` (int32 ``[B+1]``) on the device, lengths also on the host.
"""

from __future__ import annotations
from typing import List, Optional, Tuple
import torch


from ..tensor.utils import host_to_device  # noqa: F401  (re-exported: used by the fused model paths)


class PackInfo:
    """
    Layout of one packed batch.

    :ivar lens_host: int32 [B] on the host
    :ivar lens: int32 [B] on the device
    :ivar cu: int32 [B+1] on the device, prefix sums
    :ivar n: number of valid rows
    :ivar max_len: longest sequence
    :ivar gather_idx: int64 [N] index into the flattened padded ``[B*T]`` rows
    """

    def __init__(self, lens_host: torch.Tensor, device, *, padded_len: Optional[int] = None):
        lens_host = lens_host.to(torch.int32).cpu()
        self.lens_host = lens_host
        self.batch = int(lens_host.shape[0])
        self.n = int(lens_host.sum())
        self.max_len = int(lens_host.max()) if self.batch else 0
        self.padded_len = padded_len if padded_len is not None else self.max_len
        cu = torch.zeros(self.batch + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(lens_host, 0)
        self.cu_host = cu
        # one H2D copy for all layout tensors, from pinned memory so that it does not synchronise the stream
        T = self.padded_len
        b_idx = torch.repeat_interleave(torch.arange(self.batch, dtype=torch.int32), lens_host.to(torch.int64))
        t_idx = torch.arange(self.n, dtype=torch.int32) - cu[:-1][b_idx.long()]
        gather = b_idx * T + t_idx
        flat = torch.cat([lens_host, cu, b_idx, t_idx, gather])
        dev = host_to_device(flat, device)
        B, n = self.batch, self.n
        self.lens = dev[:B]
        self.cu = dev[B: 2 * B + 1]
        o = 2 * B + 1
        self.row_batch = dev[o: o + n]
        self.row_pos = dev[o + n: o + 2 * n]
        self.gather_idx = dev[o + 2 * n: o + 3 * n].long()

    def pack(self, padded: torch.Tensor) -> torch.Tensor:
        """[B, T, ...] -> [N, ...]"""
        flat = padded.reshape(padded.shape[0] * padded.shape[1], *padded.shape[2:])
        return flat.index_select(0, self.gather_idx)

    def unpack(self, rows: torch.Tensor, *, fill: float = 0.0) -> torch.Tensor:
        """[N, ...] -> [B, T, ...] (padding = fill)"""
        out = rows.new_full((self.batch * self.padded_len,) + tuple(rows.shape[1:]), fill)
        out.index_copy_(0, self.gather_idx, rows)
        return out.reshape(self.batch, self.padded_len, *rows.shape[1:])
