"""
Transformer encoder.  Parity: returnn/frontend/encoder/transformer.py.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Tuple, Union
import copy as _copy
import functools
from types import FunctionType
from ...tensor import Tensor, Dim
from ...utils.basic import NotSpecified
from ..module import Module
from ..container import Sequential
from ..linear import Linear, Embedding
from ..normalization import LayerNorm
from ..attention import SelfAttention, sinusoidal_positional_encoding
from ..dropout import dropout, dropout_broadcast_default
from ..build_from_dict import build_from_dict
from .. import math_ as _m
from ..decoder.transformer import FeedForward, make_norm

__all__ = ["TransformerEncoder", "TransformerEncoderLayer"]


class TransformerEncoderLayer(Module):
    """pre-norm block: x + SA(LN(x)); x + FF(LN(x))"""

    def __init__(self, out_dim: Dim = Dim(512, name="transformer-enc-default-out-dim"), *, ff=NotSpecified, ff_dim=NotSpecified,
                 ff_activation=NotSpecified, dropout: float = 0.1, num_heads: int = 8, self_att=None,
                 self_att_opts: Optional[Dict[str, Any]] = None, att_dropout: float = 0.1, norm=LayerNorm):
        super().__init__()
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.out_dim = out_dim
        if ff is NotSpecified:
            ff = FeedForward
        if isinstance(ff, Module):
            self.ff = _copy.deepcopy(ff)
        else:
            kw = {k: v for k, v in dict(out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, activation=ff_activation).items() if v is not NotSpecified}
            self.ff = ff(**kw) if isinstance(ff, type) else build_from_dict(ff, **kw)
        self.ff_layer_norm = make_norm(norm, out_dim)
        opts = dict(in_dim=out_dim, proj_dim=out_dim, key_dim_total=out_dim, value_dim_total=out_dim, num_heads=num_heads, att_dropout=att_dropout)
        if self_att_opts:
            opts.update(self_att_opts)
        if self_att is None:
            self.self_att = SelfAttention(**opts)
        elif isinstance(self_att, type):
            self.self_att = self_att(**opts)
        elif isinstance(self_att, dict):
            self.self_att = build_from_dict(self_att, **{k: v for k, v in opts.items() if k not in self_att})
        else:
            self.self_att = self_att
        self.self_att_layer_norm = make_norm(norm, out_dim)

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        bc = self.dropout_broadcast and self.out_dim
        x = self.self_att(self.self_att_layer_norm(inp), axis=spatial_dim)
        x = dropout(x, self.dropout, axis=bc) + inp
        y = self.ff(self.ff_layer_norm(x))
        return dropout(y, self.dropout, axis=bc) + x


class TransformerEncoder(Module):
    """embedding (sparse input) or linear projection, positional encoding, N layers, final norm"""

    def __init__(self, vocab_dim: Dim, model_dim: Union[Dim, int] = Dim(512, name="transformer-enc-default-model-dim"), *,
                 num_layers: int, ff=NotSpecified, ff_dim=NotSpecified, ff_activation=NotSpecified,
                 pos_enc=sinusoidal_positional_encoding, dropout: float = 0.1, num_heads: int = 8, att_dropout: float = 0.1,
                 norm=LayerNorm, layer=None, layer_opts: Optional[Dict[str, Any]] = None, embed_dim: Optional[Dim] = None,
                 input_embedding: bool = True, input_embedding_scale: float = None, input_dropout: float = None, sequential=Sequential):
        super().__init__()
        if isinstance(model_dim, int):
            model_dim = Dim(model_dim, name="transformer-enc-model-dim")
        self.vocab_dim = vocab_dim
        self.model_dim = model_dim
        self.out_dim = model_dim
        self.embed_dim = embed_dim
        self.input_embedding = Embedding(vocab_dim, embed_dim or model_dim) if input_embedding else None
        self.input_embedding_proj = Linear(embed_dim, model_dim, with_bias=False) if (embed_dim and embed_dim != model_dim) else None
        if pos_enc is None:
            pass
        elif isinstance(pos_enc, dict):
            pos_enc = build_from_dict(pos_enc, feat_dim=embed_dim or model_dim)
        elif isinstance(pos_enc, Module):
            pass
        elif isinstance(pos_enc, FunctionType):
            pos_enc = functools.partial(pos_enc, feat_dim=embed_dim or model_dim)
        self.pos_enc = pos_enc
        if input_embedding_scale is None:
            input_embedding_scale = model_dim.dimension ** 0.5
        self.input_embedding_scale = input_embedding_scale
        if input_dropout is None:
            input_dropout = dropout
        self.input_dropout = input_dropout
        self.dropout_broadcast = dropout_broadcast_default()
        if not layer or isinstance(layer, (dict, type)):
            opts = dict(out_dim=model_dim, ff=ff, ff_dim=ff_dim, ff_activation=ff_activation, dropout=dropout, num_heads=num_heads,
                        att_dropout=att_dropout, norm=norm)
            opts = {k: v for k, v in opts.items() if v is not NotSpecified}
            if layer_opts:
                opts.update(layer_opts)
            if not layer:
                layer = TransformerEncoderLayer(**opts)
            elif isinstance(layer, type):
                layer = layer(**opts)
            else:
                layer = build_from_dict(layer, **{k: v for k, v in opts.items() if k not in layer})
        self.layers = sequential(_copy.deepcopy(layer) for _ in range(num_layers))
        self.final_layer_norm = make_norm(norm, model_dim)

    def __call__(self, source: Tensor, *, spatial_dim: Dim, collected_outputs: Optional[Dict[str, Tensor]] = None) -> Tensor:
        x = self.input_embedding(source) * self.input_embedding_scale if self.input_embedding is not None else source
        if self.pos_enc is not None:
            x = x + self.pos_enc(spatial_dim=spatial_dim, device=x.device).copy_compatible_to_dims(x.dims) if False else x + self.pos_enc(spatial_dim=spatial_dim, device=x.device)
        x = dropout(x, self.input_dropout, axis=self.dropout_broadcast and x.feature_dim)
        if self.input_embedding_proj is not None:
            x = self.input_embedding_proj(x)
        x = self.layers(x, spatial_dim=spatial_dim, collected_outputs=collected_outputs)
        return self.final_layer_norm(x)
