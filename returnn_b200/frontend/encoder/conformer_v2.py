"""
Conformer with the frontend split off: :class:`ConformerFrontend` (subsampling prenet, bias-free projection to the model
dimension, embedding scale, input dropout; time axis shrinks) and :class:`ConformerEncoderV2` (the stack of Conformer layers
alone; time axis unchanged). ``ConformerEncoderV2(frontend(x))`` computes what :class:`ConformerEncoder` computes without a
positional encoding, and the parameter names below ``input_layer`` / ``input_projection`` / ``layers`` are the same, so a
checkpoint of one form loads into the other by prefixing.

Reference: returnn/frontend/encoder/conformer_v2.py:21 (ConformerFrontend), :86 (ConformerEncoderV2).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Tuple, Union
import copy as _copy
from ...tensor import Tensor, Dim
from ...utils.basic import NotSpecified
from ..module import Module
from ..container import Sequential
from ..linear import Linear
from ..dropout import dropout, dropout_broadcast_default
from ..build_from_dict import build_from_dict
from .base import ISeqDownsamplingEncoder, ISeqFramewiseEncoder
from .conformer import ConformerEncoderLayer, make_encoder_layer

__all__ = ["ConformerFrontend", "ConformerEncoderV2"]


class ConformerFrontend(ISeqDownsamplingEncoder):
    """``(x, in_spatial_dim) -> (y, out_spatial_dim)``: prenet, projection, scale, dropout"""

    def __init__(self, in_dim: Dim, out_dim: Dim = Dim(512, name="conformer-enc-default-out-dim"), *,
                 input_layer: Optional[Union[Dict[str, Any], Module, Callable]], input_embedding_scale: float = 1.0,
                 input_dropout: float = 0.1):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.dropout_broadcast = dropout_broadcast_default()
        if isinstance(input_layer, dict):
            input_layer = build_from_dict(input_layer, in_dim)
        elif input_layer is not None and not callable(input_layer):
            raise TypeError("%s: unexpected input_layer %r" % (self, input_layer))
        self.input_layer = input_layer
        # no prenet: the input already has the model's features and nothing is projected
        self.input_projection = Linear(input_layer.out_dim, out_dim, with_bias=False) if input_layer else None
        self.input_embedding_scale = input_embedding_scale
        self.input_dropout = input_dropout

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim) -> Tuple[Tensor, Dim]:
        x, out_spatial_dim = source, in_spatial_dim
        if self.input_layer:
            x, out_spatial_dim = self.input_layer(x, in_spatial_dim=in_spatial_dim)
        if self.input_projection:
            x = self.input_projection(x)
        if self.input_embedding_scale != 1.0:
            x = x * self.input_embedding_scale
        x = dropout(x, self.input_dropout, axis=self.dropout_broadcast and self.out_dim)
        return x, out_spatial_dim


class ConformerEncoderV2(ISeqFramewiseEncoder):
    """the Conformer layers, without any frontend: ``(x, spatial_dim) -> y`` over the same time axis"""

    def __init__(self, out_dim: Dim = Dim(512, name="conformer-enc-default-out-dim"), *, num_layers: int, ff_dim: Dim = NotSpecified,
                 ff_activation=NotSpecified, dropout: float = 0.1, conv_kernel_size: int = NotSpecified, conv_norm=NotSpecified,
                 num_heads: int = 4, att_dropout: float = 0.1, encoder_layer=None, encoder_layer_opts: Optional[Dict[str, Any]] = None,
                 sequential=Sequential):
        super().__init__()
        self.out_dim = out_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        proto = make_encoder_layer(encoder_layer, encoder_layer_opts, owner=self, out_dim=out_dim, ff_dim=ff_dim, ff_activation=ff_activation,
                                   dropout=dropout, conv_kernel_size=conv_kernel_size, conv_norm=conv_norm, num_heads=num_heads, att_dropout=att_dropout)
        self.layers = sequential(_copy.deepcopy(proto) for _ in range(num_layers))

    def __call__(self, x: Tensor, *, spatial_dim: Dim, collected_outputs: Optional[Dict[str, Tensor]] = None) -> Tensor:
        return self.layers(x, spatial_dim=spatial_dim, collected_outputs=collected_outputs)
