"""
Two-dimensional LSTM (one scan direction, from the top-left corner) over a [T, S] grid per batch entry, e.g. a target x source
plane. Each cell sees the cell above, ``(t - 1, s)``, and the cell to the left, ``(t, s - 1)``; their cell states are mixed by a
fifth gate ``lambda``:

    z(t, s) = x(t, s) W + b + h(t - 1, s) V_v + h(t, s - 1) V_h            (gates ordered input, forget, lambda, output, cell)
    c = i * tanh(z4) + f * lambda * c(t - 1, s) + f * (1 - lambda) * c(t, s - 1);    h = o * tanh(c)

All cells of an anti-diagonal are independent: the recurrence runs over the T + S - 1 diagonals, each with two batched matrix
products for the recurrent terms and one fused cell kernel (``csrc/lstm2d.cu``; plain torch ops on the CPU). The input projection
and all weight gradients are single large products outside the loop.

Reference: the TwoDLSTM op (returnn/native_op.py:1467; cell kernels :1735-1790 and :1890-1990), used by TwoDLSTMLayer
(returnn/tf/layers/rec.py:10694). Scanning from the other corners is done by flipping the input along T and / or S.
"""

from __future__ import annotations
from typing import List, Optional, Tuple
import ctypes
import torch
from . import _lib

__all__ = ["two_d_lstm", "two_d_lstm_reference"]

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and _lib.use_native(t) and hasattr(_lib.get_lib(), "rb200_lstm2d_cell_fwd")


def _diagonals(T: int, S: int, device) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    out = []
    for d in range(T + S - 1):
        t = torch.arange(max(0, d - S + 1), min(T - 1, d) + 1, device=device)
        out.append((t, d - t))
    return out


def _cell_fwd(z, c_up, c_left, mask, n: int):
    """z [R, 5n] -> (gates [R, 5n], c [R, n], h [R, n])"""
    if _native(z):
        z, c_up, c_left = z.contiguous(), c_up.contiguous(), c_left.contiguous()  # local names keep them alive until the launch is queued
        c = torch.empty_like(c_up)
        h = torch.empty_like(c_up)
        fn = _lib.bind("rb200_lstm2d_cell_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp])
        _lib.check(fn(z.data_ptr(), c_up.data_ptr(), c_left.data_ptr(), mask.data_ptr(), c.data_ptr(), h.data_ptr(),
                      z.shape[0], n, _lib.stream_ptr()), "lstm2d_cell_fwd")
        _lib.count_launch()
        return z, c, h
    i, f, lam, o, g = z.split(n, dim=1)
    i, f, lam, o, g = torch.sigmoid(i), torch.sigmoid(f), torch.sigmoid(lam), torch.sigmoid(o), torch.tanh(g)
    m = mask[:, None]
    c = (i * g + f * lam * c_up + f * (1 - lam) * c_left) * m
    return torch.cat([i, f, lam, o, g], dim=1), c, o * torch.tanh(c) * m


def _cell_bwd(gates, c, c_up, c_left, mask, dh, dc_in, n: int):
    """-> (dz [R, 5n], dc_up [R, n], dc_left [R, n])"""
    if _native(gates):
        gates, c, c_up, c_left, dh, dc_in = (t.contiguous() for t in (gates, c, c_up, c_left, dh, dc_in))
        dz = torch.empty_like(gates)
        dc_up = torch.empty_like(c)
        dc_left = torch.empty_like(c)
        fn = _lib.bind("rb200_lstm2d_cell_bwd", [_vp] * 10 + [_i64, _i32, _vp])
        _lib.check(fn(gates.data_ptr(), c.data_ptr(), c_up.data_ptr(), c_left.data_ptr(),
                      mask.data_ptr(), dh.data_ptr(), dc_in.data_ptr(), dz.data_ptr(), dc_up.data_ptr(), dc_left.data_ptr(),
                      gates.shape[0], n, _lib.stream_ptr()), "lstm2d_cell_bwd")
        _lib.count_launch()
        return dz, dc_up, dc_left
    i, f, lam, o, g = gates.split(n, dim=1)
    m = mask[:, None]
    tc = torch.tanh(c)
    dhv = dh * m
    dc = (dhv * o * (1 - tc * tc) + dc_in) * m
    dz = torch.cat([dc * g * i * (1 - i), dc * (lam * c_up + (1 - lam) * c_left) * f * (1 - f), dc * f * (c_up - c_left) * lam * (1 - lam),
                    dhv * tc * o * (1 - o), dc * i * (1 - g * g)], dim=1)
    return dz, dc * f * lam, dc * f * (1 - lam)


class _TwoDLstmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, v_h, v_v, b, mask):
        T, S, B, _ = x.shape
        n = v_h.shape[0]
        dev = x.device
        z_all = (x.reshape(T * S * B, -1).float() @ w.float() + b.float()).reshape(T, S, B, 5 * n)
        # padded by one row / column of zeros: cell (t, s) lives at [t + 1, s + 1], so "up" and "left" always exist
        hp = torch.zeros(T + 1, S + 1, B, n, device=dev)
        cp = torch.zeros(T + 1, S + 1, B, n, device=dev)
        gates_all = torch.empty(T, S, B, 5 * n, device=dev)
        diags = _diagonals(T, S, dev)
        for t, s in diags:
            nd = t.shape[0]
            h_up, h_left = hp[t, s + 1].reshape(nd * B, n), hp[t + 1, s].reshape(nd * B, n)
            z = z_all[t, s].reshape(nd * B, 5 * n) + h_up @ v_v.float() + h_left @ v_h.float()
            gates, c, h = _cell_fwd(z, cp[t, s + 1].reshape(nd * B, n), cp[t + 1, s].reshape(nd * B, n), mask[t, s].reshape(nd * B), n)
            gates_all[t, s] = gates.reshape(nd, B, 5 * n)
            hp[t + 1, s + 1] = h.reshape(nd, B, n)
            cp[t + 1, s + 1] = c.reshape(nd, B, n)
        ctx.save_for_backward(x, w, v_h, v_v, mask, gates_all, hp, cp)
        return hp[1:, 1:].clone(), cp[1:, 1:].clone()

    @staticmethod
    def backward(ctx, dy, dc_out):
        x, w, v_h, v_v, mask, gates_all, hp, cp = ctx.saved_tensors
        T, S, B, _ = x.shape
        n = v_h.shape[0]
        dev = x.device
        dhp = torch.zeros(T + 1, S + 1, B, n, device=dev)
        dcp = torch.zeros(T + 1, S + 1, B, n, device=dev)
        dhp[1:, 1:] = dy.float()
        if dc_out is not None:
            dcp[1:, 1:] = dc_out.float()
        dz_all = torch.empty(T, S, B, 5 * n, device=dev)
        for t, s in reversed(_diagonals(T, S, dev)):
            nd = t.shape[0]
            dz, dc_up, dc_left = _cell_bwd(gates_all[t, s].reshape(nd * B, 5 * n), cp[t + 1, s + 1].reshape(nd * B, n), cp[t, s + 1].reshape(nd * B, n),
                                           cp[t + 1, s].reshape(nd * B, n), mask[t, s].reshape(nd * B), dhp[t + 1, s + 1].reshape(nd * B, n),
                                           dcp[t + 1, s + 1].reshape(nd * B, n), n)
            dz_all[t, s] = dz.reshape(nd, B, 5 * n)
            # distinct (t, s) per diagonal: plain indexed accumulation has no duplicates
            dhp[t, s + 1] += (dz @ v_v.float().t()).reshape(nd, B, n)
            dhp[t + 1, s] += (dz @ v_h.float().t()).reshape(nd, B, n)
            dcp[t, s + 1] += dc_up.reshape(nd, B, n)
            dcp[t + 1, s] += dc_left.reshape(nd, B, n)
        dz2 = dz_all.reshape(T * S * B, 5 * n)
        x2 = x.reshape(T * S * B, -1).float()
        dx = (dz2 @ w.float().t()).reshape(x.shape).to(x.dtype)
        dw = (x2.t() @ dz2).to(w.dtype)
        db = dz2.sum(dim=0).to(w.dtype)
        dv_v = (hp[:-1, 1:].reshape(T * S * B, n).t() @ dz2).to(v_v.dtype)
        dv_h = (hp[1:, :-1].reshape(T * S * B, n).t() @ dz2).to(v_h.dtype)
        return dx, dw, dv_h, dv_v, db, None


def two_d_lstm(x: torch.Tensor, w: torch.Tensor, v_h: torch.Tensor, v_v: torch.Tensor, b: torch.Tensor,
               sizes: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    :param x: [T, S, B, n_in] input grid
    :param w: [n_in, 5n] input weights; ``v_h`` [n, 5n] from the left neighbour ``(t, s - 1)``; ``v_v`` [n, 5n] from the upper
        neighbour ``(t - 1, s)``; ``b`` [5n]. Gate order along 5n: input, forget, lambda, output, cell input.
    :param sizes: [B, 2] int (height <= T, width <= S) of every batch entry; cells outside produce zeros and pass no state on
    :return: (h [T, S, B, n], c [T, S, B, n]); the final state of entry b is ``c[sizes[b, 0] - 1, sizes[b, 1] - 1, b]``
    """
    T, S, B, _ = x.shape
    dev = x.device
    if sizes is None:
        mask = torch.ones(T, S, B, device=dev)
    else:
        sz = sizes.to(dev)
        mask = ((torch.arange(T, device=dev)[:, None, None] < sz[None, None, :, 0]) & (torch.arange(S, device=dev)[None, :, None] < sz[None, None, :, 1])).float()
    return _TwoDLstmFn.apply(x, w, v_h, v_v, b, mask.contiguous())


def two_d_lstm_reference(x, w, v_h, v_v, b, sizes=None):
    """cell by cell with plain autograd ops (test oracle)"""
    T, S, B, _ = x.shape
    n = v_h.shape[0]
    h = [[None] * S for _ in range(T)]
    c = [[None] * S for _ in range(T)]
    zero = torch.zeros(B, n, dtype=x.dtype, device=x.device)
    for t in range(T):
        for s in range(S):
            h_up, c_up = (h[t - 1][s], c[t - 1][s]) if t > 0 else (zero, zero)
            h_left, c_left = (h[t][s - 1], c[t][s - 1]) if s > 0 else (zero, zero)
            z = x[t, s] @ w + b + h_up @ v_v + h_left @ v_h
            i, f, lam, o, g = z.split(n, dim=1)
            i, f, lam, o, g = torch.sigmoid(i), torch.sigmoid(f), torch.sigmoid(lam), torch.sigmoid(o), torch.tanh(g)
            m = torch.ones(B, 1, dtype=x.dtype, device=x.device)
            if sizes is not None:
                m = ((t < sizes[:, 0]) & (s < sizes[:, 1])).to(x.dtype).to(x.device)[:, None]
            c[t][s] = (i * g + f * lam * c_up + f * (1 - lam) * c_left) * m
            h[t][s] = o * torch.tanh(c[t][s]) * m
    return torch.stack([torch.stack(r) for r in h]), torch.stack([torch.stack(r) for r in c])
