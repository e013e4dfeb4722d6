"""
Attention ops on ``[N, H, T, D]`` blocks (N = flattened batch dims).

- :func:`sdpa`: softmax(q k^T * scale) v with key-length masking, optional causal mask and dropout.
- :func:`rel_pos_attention`: Transformer-XL relative-position attention,
  ``score[i,j] = ((q_i+u).k_j + (q_i+v).p[j-i+T-1]) * scale``.

Native path: see :mod:`returnn_b200.ops.attention_native`; the functions below fall back to the torch math, which
is also the oracle for the kernel tests.
"""

from __future__ import annotations
from typing import Optional
import torch


def sdpa_reference(q, k, v, *, kv_lens=None, scale: float, causal: bool = False, dropout_p: float = 0.0):
    """plain torch: q [.., Tq, D], k [.., Tk, D], v [.., Tk, Dv], kv_lens [..] (leading dims like q without heads allowed)"""
    scores = torch.matmul(q, k.transpose(-1, -2)) * scale
    Tq, Tk = scores.shape[-2], scores.shape[-1]
    neg = torch.finfo(scores.dtype).min if scores.dtype != torch.bfloat16 else -1e30
    if kv_lens is not None:
        lens = kv_lens
        while lens.dim() < scores.dim() - 2:
            lens = lens.unsqueeze(-1)
        mask = torch.arange(Tk, device=q.device) < lens.unsqueeze(-1).unsqueeze(-1)
        scores = torch.where(mask, scores, torch.full((), neg, dtype=scores.dtype, device=scores.device))
    if causal:
        # query i (aligned to the end of the keys) sees keys <= i + (Tk - Tq)
        qi = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
        kj = torch.arange(Tk, device=q.device)[None, :]
        scores = torch.where(kj <= qi, scores, torch.full((), neg, dtype=scores.dtype, device=scores.device))
    w = torch.softmax(scores.float(), dim=-1).to(q.dtype)
    if dropout_p:
        w = torch.nn.functional.dropout(w, dropout_p, training=True)
    return torch.matmul(w, v)


def sdpa(q, k, v, *, kv_lens: Optional[torch.Tensor] = None, scale: float, causal: bool = False, dropout_p: float = 0.0):
    """scaled dot-product attention; leading dims of q/k/v must match (kv_lens covers the leading dims it has)"""
    if q.is_cuda:
        from . import attention_native as _n

        if _n.available(q, k, v) and _n.supports_sdpa(q, k, v, causal):
            return _n.sdpa(q, k, v, kv_lens=kv_lens, scale=scale, causal=causal, dropout_p=dropout_p)
    return sdpa_reference(q, k, v, kv_lens=kv_lens, scale=scale, causal=causal, dropout_p=dropout_p)


def rel_pos_attention_reference(q, k, v, pos, u, vb, lens, *, scale: float, dropout_p: float = 0.0):
    """
    :param q, k: [N, H, T, D]; v: [N, H, T, Dv]
    :param pos: [H, 2T-1, D] projected relative position embeddings; index r <-> distance r-(T-1)
    :param u, vb: [H, D] biases or None
    :param lens: [N] int or None
    """
    N, H, T, D = q.shape
    qu = q + u[None, :, None, :].to(q.dtype) if u is not None else q
    qv = q + vb[None, :, None, :].to(q.dtype) if vb is not None else q
    ac = torch.matmul(qu, k.transpose(-1, -2))
    bd_full = torch.matmul(qv, pos.to(q.dtype).transpose(-1, -2).unsqueeze(0))  # [N,H,T,2T-1]
    qi = torch.arange(T, device=q.device)[:, None]
    kj = torch.arange(T, device=q.device)[None, :]
    idx = (kj - qi + T - 1).expand(N, H, T, T)
    bd = torch.gather(bd_full, -1, idx)
    scores = (ac + bd) * scale
    if lens is not None:
        mask = torch.arange(T, device=q.device)[None, :] < lens[:, None]
        scores = torch.where(mask[:, None, None, :], scores, torch.full((), -1e30, dtype=scores.dtype, device=scores.device))
    w = torch.softmax(scores.float(), dim=-1).to(q.dtype)
    if dropout_p:
        w = torch.nn.functional.dropout(w, dropout_p, training=True)
    return torch.matmul(w, v)


def rel_pos_attention(q, k, v, pos, u, vb, lens, *, scale: float, dropout_p: float = 0.0):
    """relative-position self-attention, see module docstring"""
    if q.is_cuda:
        from . import attention_native as _n

        if _n.available(q, k, v) and _n.supports_rel_pos(q, k, v, pos):
            return _n.rel_pos_attention(q, k, v, pos, u, vb, lens, scale=scale, dropout_p=dropout_p)
    return rel_pos_attention_reference(q, k, v, pos, u, vb, lens, scale=scale, dropout_p=dropout_p)
