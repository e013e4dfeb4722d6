"""
Bindings of the fused attention kernels (``csrc/attention.cu``). Until a shape is supported by a kernel,
``supports_*`` returns False and the caller uses the torch math.
"""

from __future__ import annotations
import torch
from . import _lib


def available(*tensors) -> bool:
    """library present with attention entry points, bf16 inputs"""
    lib = _lib.get_lib()
    if lib is None or not hasattr(lib, "rb200_relpos_att_fwd"):
        return False
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


def supports_sdpa(q, k, v, causal: bool) -> bool:
    """shapes handled by the sdpa kernel"""
    return False


def supports_rel_pos(q, k, v, pos) -> bool:
    """shapes handled by the rel-pos kernel"""
    return False


def sdpa(q, k, v, *, kv_lens, scale, causal, dropout_p):
    """fused sdpa"""
    raise NotImplementedError


def rel_pos_attention(q, k, v, pos, u, vb, lens, *, scale, dropout_p):
    """fused rel-pos attention"""
    raise NotImplementedError


def supports_packed(num_heads: int, head_dim: int, max_len: int) -> bool:
    """shapes handled by the packed rel-pos kernel"""
    return False


def rel_pos_attention_packed(qkv, pos, u, v, pack, *, num_heads, head_dim, scale, dropout_p):
    """fused packed rel-pos attention"""
    raise NotImplementedError
