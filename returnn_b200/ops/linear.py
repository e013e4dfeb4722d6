"""
Linear layer op: ``y = x @ W (+ bias) (+ activation)`` with ``W`` stored ``[in, out]``.

On B200 (bf16 activations): forward and both backward GEMMs run on the tcgen05 GEMM kernel
(:mod:`returnn_b200.ops.gemm`) with bias/activation fused into the epilogue. Elsewhere: ``torch.matmul``.
"""

from __future__ import annotations
from typing import Optional
import torch
from . import _lib


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, activation: Optional[str] = None) -> torch.Tensor:
    """
    :param x: [..., in]
    :param weight: [in, out]
    :param bias: [out]
    :param activation: None, "relu", "silu", "gelu"
    """
    if x.is_cuda and x.dtype == torch.bfloat16 or (x.is_cuda and torch.is_autocast_enabled() and x.is_floating_point()):
        from . import gemm as _gemm

        if _gemm.available(x) and _gemm.ENABLED and x.shape[-1] % 8 == 0 and weight.shape[1] % 8 != 0 and weight.shape[1] >= 64 and activation in (
                None, "relu"):
            # An output width off the 16-byte pitch rule (a vocabulary of 10001 classes): zero columns up to the next multiple of 8, the own
            # GEMM on that, and the extra outputs cut off again. The padded copy of the weight costs a few microseconds; the library's path
            # for such widths runs at a tenth of the tensor-core rate. (Activations other than relu could map the zero columns to non-zero
            # values, which the cut removes anyway, but are left to the library path to keep this rule simple.)
            n = weight.shape[1]
            pad = -(-n // 8) * 8 - n
            w_p = torch.nn.functional.pad(weight, (0, pad))
            b_p = torch.nn.functional.pad(bias, (0, pad)) if bias is not None else None
            return _gemm.linear_bf16(x, w_p, b_p, activation)[..., :n]
        if _gemm.available(x) and _gemm.ENABLED and x.shape[-1] % 8 == 0 and weight.shape[1] % 8 == 0:
            if x.requires_grad and torch.is_grad_enabled() and weight.requires_grad:
                # parameters of a flat arena (fused AdamW): read the bf16 copy the optimizer maintains instead of casting the fp32
                # weight in every step, and add the weight / bias gradients straight into the arena
                from ..parallel import arena as _arena

                ar = _arena.find_arena(weight)
                if ar is not None:
                    y = _gemm.linear_arena(x, weight, bias, activation, ar)
                    if y is not None:
                        return y
            return _gemm.linear_bf16(x, weight, bias, activation)
    w = weight
    if not torch.is_autocast_enabled() and w.dtype != x.dtype:
        w = w.to(x.dtype)
        bias = bias.to(x.dtype) if bias is not None else None
    if bias is not None and x.dim() == 2 and activation is None and not torch.is_autocast_enabled():
        return torch.addmm(bias, x, w)
    y = torch.matmul(x, w)
    if bias is not None:
        y = y + bias
    if activation is not None:
        y = _ACT[activation](y)
    return y


_ACT = {
    "relu": torch.relu,
    "silu": torch.nn.functional.silu,
    "swish": torch.nn.functional.silu,
    "gelu": torch.nn.functional.gelu,
}
