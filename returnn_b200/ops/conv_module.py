"""
Conformer convolution module core on packed rows: ``GLU -> depthwise conv (k taps, "same") -> BatchNorm -> SiLU``.

``x [N, 2C]`` -> ``[N, C]``. The depthwise conv runs along time inside each sequence (zero outside the sequence,
padding as in ``rf.Conv1d(padding="same")``: ``(k-1)//2`` taps to the left). BatchNorm statistics are taken over the
valid frames only (masked statistics); running statistics are updated in training.

On B200: fused kernels (``csrc/conv_module.cu``); otherwise torch ops on the unpacked batch.
"""

from __future__ import annotations
import torch
import torch.nn.functional as F


def glu_dwconv_bn_silu(x: torch.Tensor, filt: torch.Tensor, bias, bn, pack, *, training: bool) -> torch.Tensor:
    """
    :param x: [N, 2C]
    :param filt: [C, 1, K] depthwise filter
    :param bias: [C] or None
    :param bn: rf.BatchNorm (gamma, beta, running_mean, running_variance, eps, momentum)
    """
    if x.is_cuda:
        from . import conv_module_native as _n

        if _n.available(x) and _n.supports(x.shape[1] // 2, filt.shape[-1]):
            return _n.glu_dwconv_bn_silu(x, filt, bias, bn, pack, training=training)
    C = x.shape[1] // 2
    K = filt.shape[-1]
    a, g = x[:, :C], x[:, C:]
    h = a * torch.sigmoid(g)
    hp = pack.unpack(h).transpose(1, 2)  # [B, C, T]
    left = (K - 1) // 2
    hp = F.pad(hp, [left, K - 1 - left])
    y = F.conv1d(hp, filt.to(hp.dtype), bias.to(hp.dtype) if bias is not None else None, groups=C)
    y = pack.pack(y.transpose(1, 2))  # [N, C]
    yf = y.float()
    if training or bn.running_mean is None:
        mean = yf.mean(dim=0)
        var = (yf - mean).square().mean(dim=0)
        if bn.running_mean is not None:
            with torch.no_grad():
                bn.running_mean.raw_tensor.lerp_(mean.detach().to(bn.running_mean.raw_tensor.dtype), bn.momentum)
                bn.running_variance.raw_tensor.lerp_(var.detach().to(bn.running_variance.raw_tensor.dtype), bn.momentum)
    else:
        mean = bn.running_mean.raw_tensor.float()
        var = bn.running_variance.raw_tensor.float()
    z = (yf - mean) * torch.rsqrt(var + bn.eps)
    if bn.affine:
        z = z * bn.gamma.raw_tensor.float() + bn.beta.raw_tensor.float()
    return F.silu(z).to(x.dtype)
