"""
Transformer decoder (causal self-attention, optional cross-attention, feed-forward), usable for whole sequences
(training) and step-wise with state (search).

Parity: returnn/frontend/decoder/transformer.py:29-568 (TransformerDecoder, TransformerDecoderLayer :302,
FeedForward :430, FeedForwardGated :484, make_norm :540). ``share_embedding`` defaults to True for
behavior_version >= 20.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Sequence, Tuple, Union
import copy as _copy
import functools
from types import FunctionType
from ...tensor import Tensor, Dim, single_step_dim
from ...utils.basic import NotSpecified, BehaviorVersion
from ..module import Module
from ..container import Sequential
from ..state import State
from ..linear import Linear, Embedding
from ..normalization import LayerNorm
from ..attention import CausalSelfAttention, CrossAttention, sinusoidal_positional_encoding
from ..dropout import dropout, dropout_broadcast_default
from ..build_from_dict import build_from_dict
from .. import math_ as _m
from .. import array_ as _a

__all__ = ["TransformerDecoder", "TransformerDecoderLayer", "FeedForward", "FeedForwardGated", "make_norm"]


class TransformerDecoder(Module):
    """Transformer decoder"""

    def __init__(self, encoder_dim: Optional[Dim], vocab_dim: Dim,
                 model_dim: Union[Dim, int] = Dim(512, name="transformer-dec-default-model-dim"), *, num_layers: int,
                 ff=NotSpecified, ff_dim=NotSpecified, ff_activation=NotSpecified, pos_enc=sinusoidal_positional_encoding,
                 dropout: float = 0.1, num_heads: int = 8, att_dropout: float = 0.1, norm=LayerNorm, layer=None,
                 layer_opts: Optional[Dict[str, Any]] = None, embed_dim: Optional[Dim] = None, share_embedding: bool = None,
                 input_embedding: bool = True, input_embedding_scale: float = None, input_dropout: float = None,
                 logits_with_bias: bool = False, sequential=Sequential, **compat_kwargs):
        super().__init__()
        if compat_kwargs:
            if "decoder_layer" in compat_kwargs:
                assert layer is None
                layer = compat_kwargs.pop("decoder_layer")
            if "decoder_layer_opts" in compat_kwargs:
                assert layer_opts is None
                layer_opts = compat_kwargs.pop("decoder_layer_opts")
            if compat_kwargs:
                raise TypeError("unexpected kwargs %r" % (compat_kwargs,))
        if not isinstance(vocab_dim, Dim):
            raise TypeError("TransformerDecoder: unexpected vocab_dim %r" % (vocab_dim,))
        if isinstance(model_dim, int):
            model_dim = Dim(model_dim, name="transformer-dec-model-dim")
        self.encoder_dim = encoder_dim
        self.vocab_dim = vocab_dim
        self.model_dim = model_dim
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
        else:
            raise TypeError("unexpected pos_enc type %r" % (pos_enc,))
        self.pos_enc = pos_enc
        if share_embedding is None:
            if embed_dim and embed_dim != model_dim:
                share_embedding = False
            elif BehaviorVersion.get() < 20:
                share_embedding = False
            else:
                share_embedding = True
        if input_embedding_scale is None:
            input_embedding_scale = model_dim.dimension ** 0.5
        self.input_embedding_scale = input_embedding_scale
        if input_dropout is None:
            input_dropout = dropout
        self.input_dropout = input_dropout
        if not layer or isinstance(layer, (dict, type)):
            opts = dict(encoder_dim=encoder_dim, out_dim=model_dim, ff=ff, ff_dim=ff_dim, ff_activation=ff_activation,
                        dropout=dropout, num_heads=num_heads, att_dropout=att_dropout, norm=norm)
            opts = {k: v for k, v in opts.items() if v is not NotSpecified}
            if layer_opts:
                opts.update(layer_opts)
            if not layer:
                layer = TransformerDecoderLayer(**opts)
            elif isinstance(layer, type):
                layer = layer(**opts)
            else:
                layer = build_from_dict(layer, **{k: v for k, v in opts.items() if k not in layer})
        elif not callable(layer):
            raise TypeError("%s: invalid non-callable layer %r" % (self, layer))
        self.layers = sequential(_copy.deepcopy(layer) for _ in range(num_layers))
        self.final_layer_norm = make_norm(norm, model_dim)
        self.logits = Linear(model_dim, vocab_dim, with_bias=logits_with_bias)
        if share_embedding:
            assert self.input_embedding is not None and not (embed_dim and embed_dim != model_dim)
            assert not logits_with_bias, "logits_with_bias=False expected with share_embedding"
            # the SAME parameter under both names (dims [vocab, model]; Linear multiplies by it transposed): the state dict then has
            # "input_embedding.weight" and "logits.weight" over one storage, as in the reference (decoder/transformer.py:192-197)
            self.logits.weight = self.input_embedding.weight
        self.share_embedding = share_embedding

    def default_initial_state(self, *, batch_dims: Sequence[Dim]) -> State:
        """initial state: per-layer states and the position counter"""
        from ..const import zeros

        state = State({k: v.default_initial_state(batch_dims=batch_dims) for k, v in self.layers._get_modules().items()})
        state.pos = zeros((), dtype="int32", device="cpu")
        return state

    def transform_encoder(self, encoder: Tensor, *, axis: Dim) -> State:
        """per-layer cross-attention keys/values of the encoder output"""
        return State({k: v.transform_encoder(encoder, axis=axis) for k, v in self.layers._get_modules().items()})

    def __call__(self, source: Tensor, *, spatial_dim: Dim, state: State, encoder: Optional[State] = None,
                 collected_outputs: Optional[Dict[str, Tensor]] = None, output_only_last_frame: bool = False) -> Tuple[Tensor, State]:
        """
        :param source: labels (sparse) or embeddings
        :param spatial_dim: single_step_dim or the label axis
        :return: logits, new state
        """
        new_state = State()
        decoded = self.input_embedding(source) if self.input_embedding is not None else source
        if self.input_embedding_scale != 1:
            decoded = decoded * self.input_embedding_scale
        if self.pos_enc is not None:
            pe = self.pos_enc(spatial_dim=spatial_dim, offset=state.pos, device=decoded.device)
            if pe.dtype != decoded.dtype:
                pe = _a.cast(pe, decoded.dtype)
            decoded = decoded + pe
        decoded = dropout(decoded, self.input_dropout)
        if self.input_embedding_proj is not None:
            decoded = self.input_embedding_proj(decoded)
        if spatial_dim == single_step_dim:
            new_state.pos = state.pos + 1
        else:
            new_state.pos = state.pos + spatial_dim.get_dim_value()
        for layer_name, layer in self.layers._get_modules().items():
            decoded, new_state[layer_name] = layer(decoded, spatial_dim=spatial_dim, state=state[layer_name],
                                                   encoder=encoder[layer_name] if encoder else None)
            if collected_outputs is not None:
                collected_outputs[layer_name] = decoded
        if output_only_last_frame and spatial_dim != single_step_dim:
            from ..dims import last_frame_position_of_dim

            decoded = _a.gather(decoded, axis=spatial_dim, indices=last_frame_position_of_dim(spatial_dim, device=decoded.device))
        decoded = self.final_layer_norm(decoded)
        logits = self.logits(decoded)
        return logits, new_state


class TransformerDecoderLayer(Module):
    """pre-norm block: causal self-attention, cross-attention (if encoder_dim), feed-forward"""

    def __init__(self, encoder_dim: Optional[Dim], out_dim: Dim = Dim(512, name="transformer-dec-default-out-dim"), *,
                 ff=NotSpecified, ff_dim=NotSpecified, ff_activation=NotSpecified, dropout: float = 0.1, num_heads: int = 8,
                 self_att=None, self_att_opts: Optional[Dict[str, Any]] = None, att_dropout: float = 0.1,
                 cross_att: Optional[Dict[str, Any]] = None, norm=LayerNorm):
        super().__init__()
        self.encoder_dim = encoder_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.out_dim = out_dim
        if ff is NotSpecified:
            ff = FeedForward
        if isinstance(ff, Module):
            ff = _copy.deepcopy(ff)
        else:
            kw = {k: v for k, v in dict(out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, activation=ff_activation).items() if v is not NotSpecified}
            if isinstance(ff, type):
                ff = ff(**kw)
            elif isinstance(ff, dict):
                ff = build_from_dict(ff, **kw)
            else:
                raise TypeError("unexpected ff type %r" % (ff,))
        self.ff = ff
        self.ff_layer_norm = make_norm(norm, out_dim)
        if self_att is None or isinstance(self_att, (dict, type)):
            opts = dict(in_dim=out_dim, proj_dim=out_dim, key_dim_total=out_dim, value_dim_total=out_dim, num_heads=num_heads, att_dropout=att_dropout)
            if self_att_opts:
                opts.update(self_att_opts)
            if self_att is None:
                self.self_att = CausalSelfAttention(**opts)
            elif isinstance(self_att, type):
                self.self_att = self_att(**opts)
            else:
                self.self_att = build_from_dict(self_att, **opts)
        else:
            self.self_att = self_att
        self.self_att_layer_norm = make_norm(norm, out_dim)
        self.cross_att = None
        self.cross_att_layer_norm = None
        if encoder_dim is not None:
            ca_opts = dict(encoder_dim=encoder_dim, query_in_dim=out_dim, proj_dim=out_dim, key_dim_total=out_dim,
                           value_dim_total=out_dim, num_heads=num_heads, att_dropout=att_dropout)
            if cross_att:
                self.cross_att = build_from_dict(cross_att, **ca_opts)
            else:
                self.cross_att = CrossAttention(**ca_opts)
            self.cross_att_layer_norm = make_norm(norm, out_dim)

    def default_initial_state(self, *, batch_dims: Sequence[Dim]) -> State:
        """self-attention history"""
        return State(self_att=self.self_att.default_initial_state(batch_dims=batch_dims))

    def transform_encoder(self, encoder: Tensor, *, axis: Dim) -> State:
        """cross-attention keys/values"""
        assert self.cross_att is not None
        return State(cross_att=self.cross_att.transform_encoder(encoder, axis=axis))

    def __call__(self, inp: Tensor, *, spatial_dim: Dim, state: State, encoder: Optional[State] = None) -> Tuple[Tensor, State]:
        new_state = State()
        bc = self.dropout_broadcast and self.out_dim
        x_sa, new_state.self_att = self.self_att(self.self_att_layer_norm(inp), axis=spatial_dim, state=state.self_att)
        x = dropout(x_sa, self.dropout, axis=bc) + inp
        if self.cross_att is not None:
            assert encoder is not None
            x_ca = self.cross_att(self.cross_att_layer_norm(x), encoder.cross_att)
            x = dropout(x_ca, self.dropout, axis=bc) + x
        x_ff = self.ff(self.ff_layer_norm(x))
        x = dropout(x_ff, self.dropout, axis=bc) + x
        return x, new_state


class FeedForward(Module):
    """Linear -> activation -> dropout -> Linear; default activation relu, ff_dim = 4 * out_dim"""

    def __init__(self, out_dim: Dim, *, ff_dim: Optional[Union[Dim, int]] = NotSpecified, dropout: float = 0.1,
                 activation=_m.relu, with_bias: bool = True):
        super().__init__()
        if isinstance(ff_dim, int):
            ff_dim = Dim(ff_dim, name="transformer-ff-dim")
        elif ff_dim is NotSpecified or ff_dim is None:
            ff_dim = out_dim * 4
        if not isinstance(ff_dim, Dim):
            raise TypeError("FeedForward: unexpected ff_dim %r" % (ff_dim,))
        if activation is NotSpecified:
            activation = _m.relu
        elif isinstance(activation, dict):
            activation = build_from_dict(activation)
        elif not callable(activation):
            raise TypeError("unexpected activation type %r" % (activation,))
        self.out_dim = out_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.activation = activation
        self.linear_ff = Linear(out_dim, ff_dim, with_bias=with_bias)
        self.linear_out = Linear(ff_dim, out_dim, with_bias=with_bias)

    def __call__(self, inp: Tensor) -> Tensor:
        x = self.activation(self.linear_ff(inp))
        x = dropout(x, self.dropout, axis=self.dropout_broadcast and self.linear_ff.out_dim)
        return self.linear_out(x)


class FeedForwardGated(Module):
    """gated variant (e.g. SwiGLU): ``linear_out(dropout(act(a) * b))`` with ``[a, b] = linear_ff(x)``; ff_dim = 4*out*2/3"""

    def __init__(self, out_dim: Dim, *, ff_dim: Optional[Union[Dim, int]] = NotSpecified, dropout: float = 0.1,
                 activation=_m.swish, gate_activation=_m.identity, with_bias: bool = False):
        super().__init__()
        if isinstance(ff_dim, int):
            ff_dim = Dim(ff_dim, name="transformer-ff-dim")
        elif ff_dim is NotSpecified or ff_dim is None:
            ff_dim = out_dim * 4 * 2 // 3
        if activation is NotSpecified:
            activation = _m.swish
        elif isinstance(activation, dict):
            activation = build_from_dict(activation)
        self.out_dim = out_dim
        self.ff_dim = ff_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.activation = activation
        self.gate_activation = gate_activation
        self.linear_ff = Linear(out_dim, 2 * ff_dim, with_bias=with_bias)
        self.linear_out = Linear(ff_dim, out_dim, with_bias=with_bias)

    def __call__(self, inp: Tensor) -> Tensor:
        x = self.linear_ff(inp)
        x, _ = _m.gating(x, out_dim=self.ff_dim, act_func=self.activation, gate_func=self.gate_activation)
        x = dropout(x, self.dropout, axis=self.dropout_broadcast and self.ff_dim)
        return self.linear_out(x)


def make_norm(norm, out_dim: Dim):
    """norm from a class / dict / module / callable spec"""
    if isinstance(norm, type):
        return norm(out_dim)
    if isinstance(norm, dict):
        return build_from_dict(norm, out_dim)
    if isinstance(norm, Module):
        return _copy.deepcopy(norm)
    if callable(norm):
        return norm
    raise TypeError("unexpected norm type %r" % (norm,))
