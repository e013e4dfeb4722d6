"""
Sequence utilities with own kernels (``csrc/seq_util.cu``) and torch references (also the CPU path):

* :func:`chunk` / :func:`unchunk`: overlapping windows of the time axis as extra batch entries, and back (mean over overlaps)
  (returnn/native_op.py:2321 Chunking, :2478 UnChunking);
* :func:`select_by_index`: ``y[t, b] = x[t, b, idx[t, b]]`` with gradient (:2655 SubtensorBatchedIndex);
* :func:`sparse_to_dense`, :func:`max_and_argmax_sparse`, :func:`sparse_ce_softmax_and_grad`: targets given as COO lists
  ``(frame s0[i, b], class s1[i, b], weight w[i, b], mask[i, b])`` per batch entry b (:2799, :2880, :2988).
"""

from __future__ import annotations
from typing import Optional, Tuple
import ctypes
import torch
from . import _lib

__all__ = ["num_chunks", "chunk", "unchunk", "select_by_index", "sparse_to_dense", "max_and_argmax_sparse", "sparse_ce_softmax_and_grad"]

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


def _native(t: torch.Tensor, name: str) -> bool:
    return t.is_cuda and _lib.use_native(t) and hasattr(_lib.get_lib(), name)


def num_chunks(T: int, chunk_size: int, chunk_step: int) -> int:
    """windows needed to cover T frames"""
    return 1 if T <= chunk_size else -(-(T - chunk_size) // chunk_step) + 1


def chunk(x: torch.Tensor, lens: torch.Tensor, *, chunk_size: int, chunk_step: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    :param x: [T, B, D] float; ``lens`` [B] valid frames
    :return: (y [chunk_size, B * n_chunks, D], y_mask [chunk_size, B * n_chunks]); window c of sequence b is column ``b * n_chunks + c``
    """
    T, B, D = x.shape
    n = num_chunks(T, chunk_size, chunk_step)
    dev = x.device
    l32 = lens.to(dev, torch.int32).contiguous()
    if _native(x, "rb200_chunk") and x.dtype == torch.float32:
        y = torch.empty(chunk_size, B * n, D, dtype=torch.float32, device=dev)
        m = torch.empty(chunk_size, B * n, dtype=torch.float32, device=dev)
        fn = _lib.bind("rb200_chunk", [_vp, _vp] + [_i32] * 6 + [_vp, _vp, _vp])
        x = x.contiguous()  # (a local name keeps the tensor alive until the launch is queued)
        _lib.check(fn(x.data_ptr(), l32.data_ptr(), T, B, D, chunk_size, chunk_step, n, y.data_ptr(), m.data_ptr(), _lib.stream_ptr()), "chunk")
        _lib.count_launch()
        return y, m
    ot = torch.arange(chunk_size, device=dev)[:, None, None]
    c = torch.arange(n, device=dev)[None, None, :]
    t = c * chunk_step + ot  # [size, 1, n]
    ok = (t < T) & (t < l32[None, :, None])  # [size, B, n]
    tt = t.clamp(max=T - 1).expand(chunk_size, B, n)
    bb = torch.arange(B, device=dev)[None, :, None].expand(chunk_size, B, n)
    y = x[tt, bb] * ok[..., None].to(x.dtype)
    return y.reshape(chunk_size, B * n, D), ok.to(torch.float32).reshape(chunk_size, B * n)


def unchunk(y: torch.Tensor, y_mask: torch.Tensor, *, T: int, B: int, chunk_size: int, chunk_step: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    inverse of :func:`chunk`; frames that several windows cover get the mean of their values.

    :return: (x [T, B, D], x_mask [T, B], factors [T, B] = 1 / number of windows that covered the frame)
    """
    D = y.shape[2]
    n = y.shape[1] // B
    dev = y.device
    if _native(y, "rb200_unchunk") and y.dtype == torch.float32:
        x = torch.empty(T, B, D, dtype=torch.float32, device=dev)
        xm = torch.empty(T, B, dtype=torch.float32, device=dev)
        fac = torch.empty(T, B, dtype=torch.float32, device=dev)
        fn = _lib.bind("rb200_unchunk", [_vp, _vp] + [_i32] * 6 + [_vp, _vp, _vp, _vp])
        y, y_mask = y.contiguous(), y_mask.float().contiguous()
        _lib.check(fn(y.data_ptr(), y_mask.data_ptr(), T, B, D, chunk_size, chunk_step, n, x.data_ptr(), xm.data_ptr(),
                      fac.data_ptr(), _lib.stream_ptr()), "unchunk")
        _lib.count_launch()
        return x, xm, fac
    acc = torch.zeros(T + chunk_size + chunk_step * n, B, D, dtype=y.dtype, device=dev)
    cnt = torch.zeros(T + chunk_size + chunk_step * n, B, dtype=y.dtype, device=dev)
    y4 = y.reshape(chunk_size, B, n, D)
    m3 = y_mask.reshape(chunk_size, B, n).to(y.dtype)
    for c in range(n):
        acc[c * chunk_step: c * chunk_step + chunk_size] += y4[:, :, c] * m3[:, :, c, None]
        cnt[c * chunk_step: c * chunk_step + chunk_size] += m3[:, :, c]
    acc, cnt = acc[:T], cnt[:T]
    x = torch.where(cnt[..., None] > 0, acc / cnt.clamp_min(1)[..., None], torch.zeros_like(acc))
    return x, (cnt > 0).to(torch.float32), torch.where(cnt > 0, 1.0 / cnt.clamp_min(1), torch.ones_like(cnt)).to(torch.float32)


class _SelectFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx):
        D = x.shape[-1]
        rows = x.numel() // D
        y = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
        fn = _lib.bind("rb200_select_by_index", [_vp, _vp, _i64, _i32, _vp, _vp])
        _lib.check(fn(x.data_ptr(), idx.data_ptr(), rows, D, y.data_ptr(), _lib.stream_ptr()), "select_by_index")
        _lib.count_launch()
        ctx.save_for_backward(idx)
        ctx.D = D
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        D = ctx.D
        dx = torch.empty(tuple(dy.shape) + (D,), dtype=torch.float32, device=dy.device)
        fn = _lib.bind("rb200_select_by_index_bwd", [_vp, _vp, _i64, _i32, _vp, _vp])
        dy = dy.contiguous().float()
        _lib.check(fn(dy.data_ptr(), idx.data_ptr(), dy.numel(), D, dx.data_ptr(), _lib.stream_ptr()), "select_by_index_bwd")
        _lib.count_launch()
        return dx, None


def select_by_index(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``y[...] = x[..., idx[...]]`` (0 where the index is out of range); gradient flows to the selected entries"""
    if _native(x, "rb200_select_by_index") and x.dtype == torch.float32:
        return _SelectFn.apply(x.contiguous(), idx.to(torch.int32).contiguous())
    D = x.shape[-1]
    ok = (idx >= 0) & (idx < D)
    return torch.gather(x, -1, idx.long().clamp(0, D - 1).unsqueeze(-1)).squeeze(-1) * ok.to(x.dtype)


def sparse_to_dense(s0: torch.Tensor, s1: torch.Tensor, weight: torch.Tensor, mask: torch.Tensor, *, T: int, D: int,
                    initial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``W[s0[i, b], b, s1[i, b]] += weight[i, b]`` for every unmasked entry; ``W`` starts from ``initial`` [T, B, D] or zeros"""
    n, B = s0.shape
    dev = weight.device
    out = initial.clone().float().contiguous() if initial is not None else torch.zeros(T, B, D, dtype=torch.float32, device=dev)
    if _native(weight, "rb200_sparse_to_dense"):
        fn = _lib.bind("rb200_sparse_to_dense", [_vp, _vp, _vp, _vp] + [_i32] * 4 + [_vp, _vp])
        s0_, s1_, w_, m_ = s0.to(torch.int32).contiguous(), s1.to(torch.int32).contiguous(), weight.float().contiguous(), mask.float().contiguous()
        _lib.check(fn(s0_.data_ptr(), s1_.data_ptr(), w_.data_ptr(), m_.data_ptr(), n, T, B, D, out.data_ptr(), _lib.stream_ptr()), "sparse_to_dense")
        _lib.count_launch()
        return out
    b = torch.arange(B, device=dev)[None, :].expand(n, B)
    ok = (mask > 0.1) & (s0 >= 0) & (s0 < T) & (s1 >= 0) & (s1 < D)
    out.index_put_((s0.long()[ok], b[ok], s1.long()[ok]), weight.float()[ok], accumulate=True)
    return out


def max_and_argmax_sparse(s0: torch.Tensor, s1: torch.Tensor, weight: torch.Tensor, mask: torch.Tensor, *, T: int,
                          init_max: float = float("-inf")) -> Tuple[torch.Tensor, torch.Tensor]:
    """per frame (t, b) the largest weight among its COO entries and that entry's class; frames without entries: (init_max, 0)"""
    n, B = s0.shape
    dev = weight.device
    out_max = torch.full((T, B), init_max, dtype=torch.float32, device=dev)
    out_arg = torch.zeros(T, B, dtype=torch.int32, device=dev)
    if _native(weight, "rb200_max_argmax_sparse"):
        best = torch.zeros(T * B, dtype=torch.int64, device=dev)
        fn = _lib.bind("rb200_max_argmax_sparse", [_vp, _vp, _vp, _vp] + [_i32] * 3 + [_vp, _vp, _vp, _vp])
        s0_, s1_, w_, m_ = s0.to(torch.int32).contiguous(), s1.to(torch.int32).contiguous(), weight.float().contiguous(), mask.float().contiguous()
        _lib.check(fn(s0_.data_ptr(), s1_.data_ptr(), w_.data_ptr(), m_.data_ptr(), n, T, B, best.data_ptr(), out_max.data_ptr(), out_arg.data_ptr(), _lib.stream_ptr()),
                   "max_argmax_sparse")
        _lib.count_launch(2)
        return out_max, out_arg
    for i in range(n):
        for b in range(B):
            if mask[i, b] > 0.1 and 0 <= int(s0[i, b]) < T:
                t, w = int(s0[i, b]), float(weight[i, b])
                if w > float(out_max[t, b]) or (w == float(out_max[t, b]) and int(s1[i, b]) < int(out_arg[t, b])):
                    out_max[t, b] = w
                    out_arg[t, b] = int(s1[i, b])
    return out_max, out_arg


def sparse_ce_softmax_and_grad(z: torch.Tensor, z_mask: torch.Tensor, y_t: torch.Tensor, y_i: torch.Tensor, y_w: torch.Tensor,
                               y_mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    :param z: [T, B, D] logits; ``z_mask`` [T, B]; the soft targets as COO lists ``y_t, y_i, y_w, y_mask`` each [n, B]
    :return: (ce [T, B] = - sum_i y[t, b, i] log softmax(z[t, b])[i], grad [T, B, D] = softmax(z) - y), both 0 at masked frames
    """
    T, B, D = z.shape
    n = y_t.shape[0]
    dev = z.device
    if _native(z, "rb200_sparse_ce_softmax_grad") and z.dtype == torch.float32:
        ce = torch.zeros(T, B, dtype=torch.float32, device=dev)
        grad = torch.empty(T, B, D, dtype=torch.float32, device=dev)
        lse = torch.empty(T, B, dtype=torch.float32, device=dev)
        fn = _lib.bind("rb200_sparse_ce_softmax_grad", [_vp] * 6 + [_i32] * 4 + [_vp] * 4)
        z_, zm_, yt_, yi_ = z.contiguous(), z_mask.float().contiguous(), y_t.to(torch.int32).contiguous(), y_i.to(torch.int32).contiguous()
        yw_, ym_ = y_w.float().contiguous(), y_mask.float().contiguous()
        _lib.check(fn(z_.data_ptr(), zm_.data_ptr(), yt_.data_ptr(), yi_.data_ptr(), yw_.data_ptr(), ym_.data_ptr(), n, T, B, D,
                      lse.data_ptr(), ce.data_ptr(), grad.data_ptr(), _lib.stream_ptr()), "sparse_ce_softmax_grad")
        _lib.count_launch(2)
        return ce, grad
    y = sparse_to_dense(y_t, y_i, y_w, y_mask, T=T, D=D)
    logp = torch.log_softmax(z.float(), dim=-1)
    zm = (z_mask > 0.1).to(torch.float32)
    return -(y * logp).sum(-1) * zm, (logp.exp() - y) * zm[..., None]
