"""
LSTM sequence op (gate order i, f, g, o; weights ``[4H, in]`` and ``[4H, H]``).

``lstm(x[T,B,in], lens[B], ...)``: frames ``t >= lens[b]`` give zero output and leave the state untouched;
``reverse=True`` runs every sequence from its own last frame to its first.

CUDA path: the input projection for all frames is one tcgen05 GEMM; the recurrence runs in the persistent kernel of
``csrc/lstm.cu`` (:mod:`returnn_b200.ops.lstm_native`). CPU path: torch's packed-sequence LSTM.
"""

from __future__ import annotations
from typing import Optional, Tuple
import torch


def lstm_reference(x, lens, w_ff, w_rec, bias, h0, c0, reverse: bool = False):
    """step-by-step torch implementation with explicit masking (oracle)"""
    T, B, _ = x.shape
    H = w_rec.shape[1]
    z_in = torch.matmul(x, w_ff.t().to(x.dtype))
    if bias is not None:
        z_in = z_in + bias.to(x.dtype)
    h, c = h0.to(x.dtype), c0.to(x.dtype)
    ys = [None] * T
    steps = range(T - 1, -1, -1) if reverse else range(T)
    wr = w_rec.t().to(x.dtype)
    for t in steps:
        z = z_in[t] + torch.matmul(h, wr)
        i, f, g, o = torch.chunk(z, 4, dim=-1)
        c_new = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h_new = torch.sigmoid(o) * torch.tanh(c_new)
        if lens is not None:
            m = (lens.to(x.device) > t).unsqueeze(-1)
            c = torch.where(m, c_new, c)
            h = torch.where(m, h_new, h)
            ys[t] = torch.where(m, h_new, torch.zeros_like(h_new))
        else:
            c, h = c_new, h_new
            ys[t] = h_new
    return torch.stack(ys, dim=0) if T else x.new_zeros(0, B, H), h, c


def _reverse_padded(x: torch.Tensor, lens: Optional[torch.Tensor]) -> torch.Tensor:
    """reverse each sequence within its own length; x [T,B,...]"""
    T = x.shape[0]
    if lens is None:
        return torch.flip(x, [0])
    pos = torch.arange(T, device=x.device)[:, None]
    l = lens.to(x.device).to(torch.int64)[None, :]
    idx = torch.where(pos < l, l - 1 - pos, pos)
    return torch.gather(x, 0, idx.reshape(T, -1, *([1] * (x.dim() - 2))).expand_as(x))


PERSIST_MAX_ROWS = 48  # batch rows of one launch of the persistent recurrence kernels
PERSIST_MAX_CHUNKS = 3  # beyond that the per-step executor (whose step time hardly grows with the batch) is the faster one


def _batch_chunks(x: torch.Tensor, lens: Optional[torch.Tensor], w_rec: torch.Tensor, w_rec_bw: Optional[torch.Tensor] = None):
    """
    The persistent recurrence kernels take at most :data:`PERSIST_MAX_ROWS` sequences. A larger batch is cut into nearly equal
    groups of consecutive sequences, each running in the persistent kernel over its own longest length (sequences are independent;
    the gradients of the weights add up through autograd), as long as that beats the per-step executor.

    :return: list of (b0, b1, frames) or None when the batch is not to be cut
    """
    from . import lstm_native as _n

    T, B, _ = x.shape
    n = -(-B // PERSIST_MAX_ROWS)
    if B <= PERSIST_MAX_ROWS or n > PERSIST_MAX_CHUNKS or T == 0:
        return None
    if w_rec_bw is not None and w_rec_bw.shape != w_rec.shape:
        return None
    per = -(-B // n)
    if not _n.persist_supported(x, per, w_rec):
        return None
    lens_host = lens.tolist() if (lens is not None and not lens.is_cuda) else None
    out = []
    for b0 in range(0, B, per):
        b1 = min(B, b0 + per)
        t = max(1, min(T, max(lens_host[b0:b1]))) if lens_host is not None else T
        out.append((b0, b1, t))
    return out


def _padded_hidden(x: torch.Tensor, w_rec: torch.Tensor) -> int:
    """
    The persistent recurrence kernels want a hidden size that is a multiple of 128. Other sizes are run zero-padded: units whose weights,
    bias and initial state are zero stay exactly zero (their candidate is tanh(0) = 0, so the cell never moves and h = o * tanh(0) = 0),
    so the first H units compute the same function, at the cost of the extra units, and still far below the per-step executor.

    :return: padded size to use, or 0 when the size is fine as it is or the padded problem does not fit the kernels either
    """
    from . import lstm_native as _n

    H = w_rec.shape[1]
    if H % 128 == 0 or x.shape[0] == 0:
        return 0
    Hp = -(-H // 128) * 128
    B = x.shape[1]
    if B > PERSIST_MAX_ROWS * PERSIST_MAX_CHUNKS:
        return 0
    per = -(-B // (-(-B // PERSIST_MAX_ROWS)))
    lib_ok = _n.available(x) and x.shape[-1] % 8 == 0
    if not lib_ok:
        return 0
    from . import _lib
    import ctypes

    fn = _lib.bind("rb200_blstm_supported", [ctypes.c_int, ctypes.c_int, ctypes.c_int])
    return Hp if fn(int(x.shape[0]), int(per), int(Hp)) else 0


def _pad_input(x: torch.Tensor, w_ff: torch.Tensor):
    """input width up to a multiple of 8 (the 16-byte pitch rule of the tensor maps) with zero features and zero weight columns: same product"""
    n = -(-x.shape[-1] // 8) * 8 - x.shape[-1]
    return torch.nn.functional.pad(x, (0, n)), torch.nn.functional.pad(w_ff, (0, n))


def _pad_params(w_ff, w_rec, bias, H: int, Hp: int):
    """gate-wise zero padding: [4H, in] -> [4Hp, in], [4H, H] -> [4Hp, Hp], [4H] -> [4Hp]"""
    F = torch.nn.functional
    w_ff_p = F.pad(w_ff.reshape(4, H, -1), (0, 0, 0, Hp - H)).reshape(4 * Hp, -1)
    w_rec_p = F.pad(w_rec.reshape(4, H, H), (0, Hp - H, 0, Hp - H)).reshape(4 * Hp, Hp)
    bias_p = F.pad(bias.reshape(4, H), (0, Hp - H)).reshape(4 * Hp) if bias is not None else None
    return w_ff_p, w_rec_p, bias_p


def _join_chunks(outs, T: int):
    """(y [t_c, b_c, H], h, c) per chunk -> one (y [T, B, H], h, c); frames beyond a chunk's own length are zero"""
    ys = [torch.nn.functional.pad(y, (0, 0, 0, 0, 0, T - y.shape[0])) if y.shape[0] < T else y for y, _h, _c in outs]
    return torch.cat(ys, dim=1), torch.cat([h for _y, h, _c in outs], dim=0), torch.cat([c for _y, _h, c in outs], dim=0)


def lstm(x: torch.Tensor, lens: Optional[torch.Tensor], w_ff: torch.Tensor, w_rec: torch.Tensor, bias: Optional[torch.Tensor],
         h0: torch.Tensor, c0: torch.Tensor, reverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    :param x: [T, B, in]
    :param lens: [B] int32 (on any device) or None
    :return: y [T, B, H], h_T [B, H], c_T [B, H]
    """
    if x.is_cuda and x.shape[-1] % 8:
        x, w_ff = _pad_input(x, w_ff)
    if x.is_cuda:
        from . import lstm_native as _n

        Hp = _padded_hidden(x, w_rec)
        if Hp:
            H = w_rec.shape[1]
            pad = (0, Hp - H)
            y, h, c = lstm(x, lens, *_pad_params(w_ff, w_rec, bias, H, Hp), torch.nn.functional.pad(h0, pad), torch.nn.functional.pad(c0, pad), reverse=reverse)
            return y[..., :H], h[..., :H], c[..., :H]
        if _n.available(x) and _n.supports(x, w_rec):
            chunks = _batch_chunks(x, lens, w_rec)
            if chunks:
                outs = [_n.lstm(x[:t, b0:b1], lens[b0:b1] if lens is not None else None, w_ff, w_rec, bias, h0[b0:b1], c0[b0:b1], reverse=reverse)
                        for b0, b1, t in chunks]
                return _join_chunks(outs, x.shape[0])
            return _n.lstm(x, lens, w_ff, w_rec, bias, h0, c0, reverse=reverse)
    T, B, _ = x.shape
    H = w_rec.shape[1]
    if T == 0:
        return x.new_zeros(0, B, H), h0, c0
    dt = x.dtype
    if torch.is_autocast_enabled() and x.is_cuda:
        dt = torch.get_autocast_dtype("cuda")
    ws = [w_ff.to(dt), w_rec.to(dt)]
    if bias is not None:
        ws += [bias.to(dt), torch.zeros_like(bias, dtype=dt)]
    xx = x.to(dt)
    if reverse:
        xx = _reverse_padded(xx, lens)
    if lens is not None:
        packed = torch.nn.utils.rnn.pack_padded_sequence(xx, lens.cpu().to(torch.int64), enforce_sorted=False)
        out, hT, cT = torch.lstm(packed.data, packed.batch_sizes, (h0.unsqueeze(0).to(dt), c0.unsqueeze(0).to(dt)), ws,
                                 bias is not None, 1, 0.0, torch.is_grad_enabled(), False)  # "train": cuDNN keeps what its backward needs
        y, _ = torch.nn.utils.rnn.pad_packed_sequence(
            torch.nn.utils.rnn.PackedSequence(out, packed.batch_sizes, packed.sorted_indices, packed.unsorted_indices), total_length=T)
        if packed.unsorted_indices is not None:
            hT = hT.index_select(1, packed.unsorted_indices)
            cT = cT.index_select(1, packed.unsorted_indices)
    else:
        y, hT, cT = torch.lstm(xx, (h0.unsqueeze(0).to(dt), c0.unsqueeze(0).to(dt)), ws, bias is not None, 1, 0.0, torch.is_grad_enabled(), False, False)
    if reverse:
        y = _reverse_padded(y, lens)
    return y, hT[0], cT[0]


def blstm(x: torch.Tensor, lens: Optional[torch.Tensor], fw, bw, h0_fw, c0_fw, h0_bw, c0_bw):
    """
    Both directions of a bidirectional layer over the same input.

    On the GPU the two recurrences run in ONE persistent kernel (half of the CTAs per direction, two CTAs per SM) when the
    shape allows it: a recurrence is bound by the latency of its per-step grid barrier, not by throughput, so two of them
    side by side take little more than one. Otherwise two calls of :func:`lstm`.

    :param x: [T, B, in]
    :param fw: (w_ff, w_rec, bias) of the direction that runs forward in time; ``bw``: of the reversed one
    :return: (y_fw, h_T, c_T), (y_bw, h_T, c_T)
    """
    if x.is_cuda and x.shape[-1] % 8:
        x, w_fw = _pad_input(x, fw[0])
        fw, bw = (w_fw, fw[1], fw[2]), (torch.nn.functional.pad(bw[0], (0, x.shape[-1] - bw[0].shape[1])), bw[1], bw[2])
    if x.is_cuda:
        from . import lstm_native as _n

        Hp = _padded_hidden(x, fw[1]) if fw[1].shape == bw[1].shape else 0
        if Hp:
            H = fw[1].shape[1]
            pad = (0, Hp - H)
            P = torch.nn.functional.pad
            (yf, hf, cf), (yb, hb, cb) = blstm(x, lens, _pad_params(*fw, H, Hp), _pad_params(*bw, H, Hp), P(h0_fw, pad), P(c0_fw, pad), P(h0_bw, pad),
                                               P(c0_bw, pad))
            return (yf[..., :H], hf[..., :H], cf[..., :H]), (yb[..., :H], hb[..., :H], cb[..., :H])
        if _n.blstm_supported(x, fw[1], bw[1]):
            return _n.blstm(x, lens, fw, bw, h0_fw, c0_fw, h0_bw, c0_bw)
        chunks = _batch_chunks(x, lens, fw[1], bw[1])
        if chunks:
            outs = [_n.blstm(x[:t, b0:b1], lens[b0:b1] if lens is not None else None, fw, bw, h0_fw[b0:b1], c0_fw[b0:b1], h0_bw[b0:b1], c0_bw[b0:b1])
                    for b0, b1, t in chunks]
            return _join_chunks([o[0] for o in outs], x.shape[0]), _join_chunks([o[1] for o in outs], x.shape[0])
    return (lstm(x, lens, fw[0], fw[1], fw[2], h0_fw, c0_fw, reverse=False),
            lstm(x, lens, bw[0], bw[1], bw[2], h0_bw, c0_bw, reverse=True))
