"""
Relative-position multi-head self-attention on packed rows.

Input ``qkv [N, H*3*D]`` (per head grouped as q, k, v), projected relative position embeddings
``pos [2*L-1, H*D]`` (row ``r`` = distance ``r - (L-1)``), biases ``u, v [H, D]`` and the packed layout
(``cu_seqlens``). Output ``[N, H*D]``. ``score[i,j] = ((q_i+u).k_j + (q_i+v).p[j-i]) * scale`` within each sequence.

On B200: the fused sm_100a kernel (``csrc/attention.cu``), forward and backward, without padding and without the
``[B,H,T,2T-1]`` intermediate. Otherwise: unpack to ``[B,H,T,D]`` and use the torch math.
"""

from __future__ import annotations
import torch
from . import attention as _att


def rel_pos_attention_packed(qkv: torch.Tensor, pos: torch.Tensor, u, v, pack, *, num_heads: int, head_dim: int,
                             scale: float, dropout_p: float = 0.0) -> torch.Tensor:
    """see module docstring"""
    if qkv.is_cuda:
        from . import attention_native as _n

        if _n.available(qkv) and _n.supports_packed(num_heads, head_dim, pack.max_len):
            return _n.rel_pos_attention_packed(qkv, pos, u, v, pack, num_heads=num_heads, head_dim=head_dim, scale=scale, dropout_p=dropout_p)
    N = qkv.shape[0]
    H, D = num_heads, head_dim
    x = qkv.reshape(N, H, 3, D)
    pad = pack.unpack(x)  # [B,T,H,3,D]
    T = pad.shape[1]
    q = pad[:, :, :, 0].permute(0, 2, 1, 3)
    k = pad[:, :, :, 1].permute(0, 2, 1, 3)
    vv = pad[:, :, :, 2].permute(0, 2, 1, 3)
    L = (pos.shape[0] + 1) // 2
    p = pos.reshape(2 * L - 1, H, D).permute(1, 0, 2)  # [H, 2L-1, D]
    if T != L:
        # rows r=0..2T-2 of the reference layout correspond to distances -(T-1)..T-1
        p = p[:, (L - 1) - (T - 1): (L - 1) + T]
    out = _att.rel_pos_attention_reference(q, k, vv, p, u, v, pack.lens, scale=scale, dropout_p=dropout_p)  # [B,H,T,D]
    out = out.permute(0, 2, 1, 3).reshape(out.shape[0], T, H * D)
    return pack.pack(out)
