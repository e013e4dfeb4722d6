"""
E-Branchformer layer (https://arxiv.org/abs/2210.00077): parallel self-attention and cgMLP branches, merged by a
depthwise conv + linear.  Parity: returnn/frontend/encoder/e_branchformer.py.
"""

from __future__ import annotations
from typing import Optional, Dict, Any
from ...tensor import Tensor, Dim
from ...utils.basic import NotSpecified
from ..module import Module
from ..linear import Linear
from ..conv import Conv1d
from ..normalization import LayerNorm
from ..attention import RelPosSelfAttention
from ..dropout import dropout, dropout_broadcast_default
from .. import math_ as _m
from .. import array_ as _a
from .conformer import make_ff
from ..decoder.transformer import make_norm

__all__ = ["EBranchformerLayer", "FeedForwardConvGated", "Merge"]


class FeedForwardConvGated(Module):
    """cgMLP: Linear -> GELU -> split -> (a * dwconv(LN(b))) -> Linear"""

    def __init__(self, out_dim: Dim, *, ff_dim: Optional[Dim] = None, kernel_size: int = 31, dropout: float = 0.1,
                 activation=_m.gelu, gate_activation=_m.identity, with_bias: bool = True, norm=LayerNorm):
        super().__init__()
        if ff_dim is None:
            ff_dim = 6 * out_dim
        self.out_dim = out_dim
        self.ff_dim = ff_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.activation = activation
        self.gate_activation = gate_activation
        self.linear_ff = Linear(out_dim, ff_dim, with_bias=with_bias)
        self.half = ff_dim.div_left(2)
        self.norm = make_norm(norm, self.half)
        self.conv = Conv1d(self.half, self.half, filter_size=kernel_size, groups=self.half.dimension, padding="same")
        self.linear_out = Linear(self.half, out_dim, with_bias=with_bias)

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        x = self.activation(self.linear_ff(inp))
        a, b = _a.split(x, axis=self.ff_dim, out_dims=[self.half, self.half])
        b = self.norm(b)
        b, _ = self.conv(b, in_spatial_dim=spatial_dim)
        x = a * self.gate_activation(b)
        x = dropout(x, self.dropout, axis=self.dropout_broadcast and self.half)
        return self.linear_out(x)


class Merge(Module):
    """concat both branches, add depthwise conv of the concat, project back"""

    def __init__(self, in_dim1: Dim, in_dim2: Dim, out_dim: Dim, *, merge_conv_kernel_size: int = 31):
        super().__init__()
        self.in_dim1, self.in_dim2, self.out_dim = in_dim1, in_dim2, out_dim
        self.concat_dim = in_dim1 + in_dim2
        self.depthwise_conv = Conv1d(self.concat_dim, self.concat_dim, filter_size=merge_conv_kernel_size,
                                     groups=self.concat_dim.dimension, padding="same")
        self.linear_ff = Linear(self.concat_dim, out_dim)

    def __call__(self, x1: Tensor, x2: Tensor, *, spatial_dim: Dim) -> Tensor:
        x, _ = _a.concat((x1, self.in_dim1), (x2, self.in_dim2), out_dim=self.concat_dim)
        x_conv, _ = self.depthwise_conv(x, in_spatial_dim=spatial_dim)
        return self.linear_ff(x + x_conv)


class EBranchformerLayer(Module):
    """one E-Branchformer block"""

    def __init__(self, out_dim: Dim = Dim(512, name="e-branchformer-default-out-dim"), *, ff=NotSpecified, ff_dim=NotSpecified,
                 ff_activation=NotSpecified, dropout: float = 0.1, num_heads: int = 4, self_att=None,
                 self_att_opts: Optional[Dict[str, Any]] = None, att_dropout: float = 0.1, cgmlp_ff_dim=None,
                 cgmlp_conv_kernel: int = 31, merge_conv_kernel: int = 3, norm=LayerNorm):
        super().__init__()
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.out_dim = out_dim
        self.ffn1 = make_ff(ff=ff, out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, ff_activation=ff_activation)
        self.ffn1_layer_norm = make_norm(norm, out_dim)
        self.ffn2 = make_ff(ff=ff, out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, ff_activation=ff_activation)
        self.ffn2_layer_norm = make_norm(norm, out_dim)
        opts = dict(in_dim=out_dim, proj_dim=out_dim, key_dim_total=out_dim, value_dim_total=out_dim, num_heads=num_heads, att_dropout=att_dropout)
        if self_att_opts:
            opts.update(self_att_opts)
        self.self_att = self_att if (self_att is not None and not isinstance(self_att, type)) else (self_att or RelPosSelfAttention)(**opts)
        self.self_att_layer_norm = make_norm(norm, out_dim)
        self.cgmlp = FeedForwardConvGated(out_dim, ff_dim=cgmlp_ff_dim, kernel_size=cgmlp_conv_kernel, dropout=dropout)
        self.cgmlp_layer_norm = make_norm(norm, out_dim)
        self.merge = Merge(out_dim, out_dim, out_dim, merge_conv_kernel_size=merge_conv_kernel)
        self.final_layer_norm = make_norm(norm, out_dim)

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        bc = self.dropout_broadcast and self.out_dim
        x = 0.5 * dropout(self.ffn1(self.ffn1_layer_norm(inp)), self.dropout, axis=bc) + inp
        x1 = dropout(self.self_att(self.self_att_layer_norm(x), axis=spatial_dim), self.dropout, axis=bc)
        x2 = dropout(self.cgmlp(self.cgmlp_layer_norm(x), spatial_dim=spatial_dim), self.dropout, axis=bc)
        x = dropout(self.merge(x1, x2, spatial_dim=spatial_dim), self.dropout, axis=bc) + x
        x = 0.5 * dropout(self.ffn2(self.ffn2_layer_norm(x)), self.dropout, axis=bc) + x
        return self.final_layer_norm(x)
