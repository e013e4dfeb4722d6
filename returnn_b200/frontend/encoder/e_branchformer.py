"""
E-Branchformer layer (https://arxiv.org/abs/2210.00077): parallel self-attention and cgMLP branches, merged by a
depthwise conv + linear. Meant as the ``encoder_layer`` of :class:`ConformerEncoder` / :class:`ConformerEncoderV2`.
Module and parameter names equal the reference's (returnn/frontend/encoder/e_branchformer.py:40 layer, :151 cgMLP, :248 merge),
so checkpoints interchange.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Union
import copy as _copy
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
from ..build_from_dict import build_from_dict
from .conformer import make_ff
from ..decoder.transformer import make_norm

__all__ = ["EBranchformerLayer", "FeedForwardConvGated", "Merge"]


def _make_activation(activation) -> Callable[[Tensor], Tensor]:
    if isinstance(activation, dict):
        activation = build_from_dict(activation)
    elif isinstance(activation, Module):
        activation = _copy.deepcopy(activation)
    elif isinstance(activation, type):
        activation = activation()
    if not callable(activation):
        raise TypeError("unexpected activation %r" % (activation,))
    return activation


def _make_sub_module(spec, default_cls, opts: Dict[str, Any], *pos_args, what: str):
    """``NotSpecified`` -> default class; class -> instance; dict -> build_from_dict (named keys win over ``opts``); module -> copy"""
    opts = {k: v for k, v in opts.items() if v is not NotSpecified}
    if spec is NotSpecified or spec is None:
        spec = default_cls
    if isinstance(spec, type):
        return spec(*pos_args, **opts)
    if isinstance(spec, dict):
        return build_from_dict(spec, *pos_args, **{k: v for k, v in opts.items() if k not in spec})
    if isinstance(spec, Module):
        return _copy.deepcopy(spec)
    raise TypeError("invalid %s %r (type %s)" % (what, spec, type(spec).__name__))


class FeedForwardConvGated(Module):
    """
    cgMLP, the local branch: ``Linear(D -> 2F) -> activation -> split into (g, r) -> conv_dw(norm(g)) gated with r -> dropout
    -> Linear(F -> D)``. ``ff_dim`` is F, the width of ONE of the two halves (half of ESPnet's ``cgmlp_linear_units``);
    default 3 x model dim.
    """

    def __init__(self, out_dim: Dim, *, ff_dim: Union[Dim, int] = NotSpecified, kernel_size: int = 31, dropout: float = 0.1,
                 activation=_m.gelu, gate_activation=_m.identity, with_bias: bool = True, norm=LayerNorm):
        super().__init__()
        if ff_dim is NotSpecified or ff_dim is None:
            ff_dim = out_dim * 3
        if isinstance(ff_dim, int):
            ff_dim = Dim(ff_dim, name="e-branchformer-ff-dim")
        if not isinstance(ff_dim, Dim):
            raise TypeError("FeedForwardConvGated: unexpected ff_dim %r" % (ff_dim,))
        self.out_dim = out_dim
        self.ff_dim = ff_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.activation = _make_activation(_m.gelu if activation is NotSpecified else activation)
        self.gate_activation = _make_activation(_m.identity if gate_activation is NotSpecified else gate_activation)
        self.linear_ff = Linear(out_dim, 2 * ff_dim, with_bias=with_bias)
        self.norm = make_norm(norm, ff_dim)
        self.conv = Conv1d(ff_dim, ff_dim, filter_size=kernel_size, groups=ff_dim.dimension, padding="same", with_bias=with_bias)
        self.linear_out = Linear(ff_dim, out_dim, with_bias=with_bias)

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        x = self.activation(self.linear_ff(inp))
        gate, rest = _a.split(x, axis=self.linear_ff.out_dim, out_dims=[self.ff_dim, self.ff_dim])
        gate, _ = self.conv(self.norm(gate), in_spatial_dim=spatial_dim)
        x = self.gate_activation(gate) * rest
        x = dropout(x, self.dropout, axis=self.dropout_broadcast and self.ff_dim)
        return self.linear_out(x)


class Merge(Module):
    """both branches concatenated, plus a depthwise conv of the concatenation, projected back to the model dim"""

    def __init__(self, *, in_dim1: Dim, in_dim2: Dim, out_dim: Dim, merge_conv_kernel: int = 3):
        super().__init__()
        self.in_dim1, self.in_dim2, self.out_dim = in_dim1, in_dim2, out_dim
        self.concat_in_dim = in_dim1 + in_dim2
        self.depthwise_conv_fusion = Conv1d(self.concat_in_dim, self.concat_in_dim, filter_size=merge_conv_kernel,
                                            groups=self.concat_in_dim.dimension, padding="same")
        self.merge_proj = Linear(self.concat_in_dim, out_dim)

    def __call__(self, x1: Tensor, x2: Tensor, *, spatial_dim: Dim) -> Tensor:
        x, _ = _a.concat((x1, self.in_dim1), (x2, self.in_dim2), out_dim=self.concat_in_dim)
        x_conv, _ = self.depthwise_conv_fusion(x, in_spatial_dim=spatial_dim)
        return self.merge_proj(x + x_conv)


class EBranchformerLayer(Module):
    """one E-Branchformer block: macaron FF, (self-attention || cgMLP) -> merge, macaron FF, final norm"""

    def __init__(self, out_dim: Dim = Dim(512, name="conformer-enc-default-out-dim"), *, ff=NotSpecified, ff_dim=NotSpecified,
                 ff_activation=NotSpecified, dropout: float = 0.1, num_heads: int = 4, self_att=NotSpecified, att_dropout: float = 0.1,
                 cgmlp=NotSpecified, cgmlp_ff_dim=NotSpecified, cgmlp_conv_kernel: int = 31, merge_conv_kernel: int = 3, norm=LayerNorm):
        super().__init__()
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.out_dim = out_dim
        self.ffn1 = make_ff(ff=ff, out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, ff_activation=ff_activation)
        self.ffn1_layer_norm = make_norm(norm, out_dim)
        self.ffn2 = make_ff(ff=ff, out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, ff_activation=ff_activation)
        self.ffn2_layer_norm = make_norm(norm, out_dim)
        self.self_att = _make_sub_module(self_att, RelPosSelfAttention, dict(
            in_dim=out_dim, proj_dim=out_dim, key_dim_total=out_dim, value_dim_total=out_dim, num_heads=num_heads, att_dropout=att_dropout), what="self_att")
        self.self_att_layer_norm = make_norm(norm, out_dim)
        self.cgmlp = _make_sub_module(cgmlp, FeedForwardConvGated, dict(ff_dim=cgmlp_ff_dim, kernel_size=cgmlp_conv_kernel, dropout=dropout),
                                      out_dim, what="cgmlp")
        self.cgmlp_layer_norm = make_norm(norm, out_dim)
        self.merge = Merge(in_dim1=out_dim, in_dim2=out_dim, out_dim=out_dim, merge_conv_kernel=merge_conv_kernel)
        self.final_layer_norm = make_norm(norm, out_dim)

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        bc = self.dropout_broadcast and self.out_dim
        x = 0.5 * dropout(self.ffn1(self.ffn1_layer_norm(inp)), self.dropout, axis=bc) + inp
        x1 = dropout(self.self_att(self.self_att_layer_norm(x), axis=spatial_dim), self.dropout, axis=bc)
        x2 = dropout(self.cgmlp(self.cgmlp_layer_norm(x), spatial_dim=spatial_dim), self.dropout, axis=bc)
        x = dropout(self.merge(x1, x2, spatial_dim=spatial_dim), self.dropout, axis=bc) + x
        x = 0.5 * dropout(self.ffn2(self.ffn2_layer_norm(x)), self.dropout, axis=bc) + x
        return self.final_layer_norm(x)
