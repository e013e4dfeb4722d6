"""
Rotary position embedding applied to the last axis.

Parity: returnn/torch/util/rope.py (apply_rope :15).
"""

from __future__ import annotations
import torch


def apply_rope(x: torch.Tensor, pos_enc: torch.Tensor) -> torch.Tensor:
    """
    :param x: [..., D], D even; feature pairs are (x[..., :D/2], x[..., D/2:]) ("rotate half" convention)
    :param pos_enc: broadcastable to x, [..., D] = concat(sin [D/2], cos [D/2]) of the position angles
    :return: rotated x, same shape and dtype
    """
    d = x.shape[-1]
    assert d % 2 == 0 and pos_enc.shape[-1] == d
    half = d // 2
    sin, cos = pos_enc[..., :half], pos_enc[..., half:]
    a, b = x[..., :half].float(), x[..., half:].float()
    out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    return out.to(x.dtype)
