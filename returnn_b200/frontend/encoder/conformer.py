"""
Conformer encoder (https://arxiv.org/abs/2005.08100): conv2d subsampling frontend, then blocks of
FFN(1/2) - rel-pos MHSA - conv module - FFN(1/2) - LayerNorm.

Two execution paths share one set of parameters (same checkpoint keys):

- the generic path below composes RF ops on padded ``[B, T, F]`` tensors (any configuration, any device);
- on B200, for the standard configuration, ``ConformerEncoder.__call__`` switches to the fused packed-row path of
  :mod:`returnn_b200.models.conformer_fused`.

Parity: returnn/frontend/encoder/conformer.py:22-537.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Tuple, Union
from types import FunctionType
import copy as _copy
import functools
import inspect
from ...tensor import Tensor, Dim
from ...utils.basic import NotSpecified
from .. import module as _module
from ..module import Module
from ..container import ModuleList, Sequential
from ..linear import Linear
from ..conv import Conv1d, Conv2d, make_conv_out_spatial_dims, pool2d
from ..normalization import LayerNorm, BatchNorm
from ..attention import RelPosSelfAttention
from ..dropout import dropout, dropout_broadcast_default
from ..build_from_dict import build_from_dict
from .. import math_ as _m
from .. import array_ as _a
from ..dims import replace_dim
from .base import ISeqDownsamplingEncoder
from ..decoder.transformer import FeedForward, make_norm

__all__ = ["ConformerPositionwiseFeedForward", "ConformerConvBlock", "ConformerConvSubsample", "ConformerEncoderLayer",
           "ConformerEncoder", "make_ff", "conv_norm_use_mask_default"]


class ConformerPositionwiseFeedForward(FeedForward):
    """Linear -> swish -> dropout -> Linear"""

    def __init__(self, out_dim: Dim, *, ff_dim=NotSpecified, dropout: float = 0.1, activation=_m.swish, **kwargs):
        if activation is NotSpecified:
            activation = _m.swish
        super().__init__(out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, activation=activation, **kwargs)


class ConformerConvBlock(Module):
    """pointwise conv (x2) -> GLU -> depthwise conv -> norm -> swish -> pointwise conv"""

    def __init__(self, out_dim: Dim, *, kernel_size: int, norm):
        super().__init__()
        self.out_dim = out_dim
        self.positionwise_conv1 = Linear(out_dim, 2 * out_dim)
        self.depthwise_conv = Conv1d(out_dim, out_dim, filter_size=kernel_size, groups=out_dim.dimension, padding="same")
        self.positionwise_conv2 = Linear(out_dim, out_dim)
        if not callable(norm):
            raise TypeError("%s: unexpected norm type %r" % (self, norm))
        self.norm = norm
        self._norm_wants_spatial_dim = "spatial_dim" in inspect.signature(norm.__call__ if isinstance(norm, Module) else norm).parameters

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        x_conv1 = self.positionwise_conv1(inp)
        x_act, _ = _m.gating(x_conv1)
        x_depthwise_conv, _ = self.depthwise_conv(x_act, in_spatial_dim=spatial_dim)
        if self._norm_wants_spatial_dim:
            x_normed = self.norm(x_depthwise_conv, spatial_dim=spatial_dim)
        else:
            x_normed = self.norm(x_depthwise_conv)
        x_swish = _m.swish(x_normed)
        return self.positionwise_conv2(x_swish)


class ConformerConvSubsample(ISeqDownsamplingEncoder):
    """
    Stack of Conv2d over (time, feature) with optional max-pooling / striding, then the remaining feature axis and the
    channels are merged. ESPnet Conv2dSubsampling6: ``out_dims=[D, D], filter_sizes=[3, 5], strides=[2, 3], padding="valid"``.
    """

    def __init__(self, in_dim: Dim, *, out_dims: List[Union[Dim, int]], filter_sizes: List[Union[int, Tuple[int, int]]],
                 strides: Optional[List[Union[int, Tuple[int, int]]]] = None, pool_sizes: Optional[List[Tuple[int, int]]] = None,
                 activation: Callable[[Tensor], Tensor] = _m.relu, padding: str = "same"):
        super().__init__()
        self.pool_sizes = pool_sizes
        self.activation = activation
        self.conv_layers = ModuleList()
        if strides is None:
            strides = [1] * len(out_dims)
        assert len(out_dims) == len(filter_sizes) == len(strides) > 0
        self._dummy_in_dim = Dim(1, name="conv_dummy_in")
        self.in_dim = in_dim
        prev_out_dim = self._dummy_in_dim
        second_spatial_dim = in_dim
        self._strides2 = []
        for i, (filter_size, stride, out_dim) in enumerate(zip(filter_sizes, strides, out_dims)):
            if isinstance(out_dim, int):
                out_dim = Dim(out_dim, name="conv_out_%i" % i)
            conv = Conv2d(prev_out_dim, out_dim, filter_size=filter_size, strides=stride, padding=padding)
            self.conv_layers.append(conv)
            st = (stride, stride) if isinstance(stride, int) else tuple(stride)
            self._strides2.append(st)
            (second_spatial_dim,) = make_conv_out_spatial_dims([second_spatial_dim], filter_size=conv.filter_size[1].dimension,
                                                               strides=st[1], padding=padding)
            if self.pool_sizes and i < len(self.pool_sizes):
                (second_spatial_dim,) = make_conv_out_spatial_dims([second_spatial_dim], filter_size=self.pool_sizes[i][1],
                                                                   strides=self.pool_sizes[i][1], padding="same")
            prev_out_dim = out_dim
        self._final_second_spatial_dim = second_spatial_dim
        self.out_dim = second_spatial_dim * prev_out_dim
        self.downsample_factor = 1
        for i, st in enumerate(self._strides2):
            self.downsample_factor *= st[0]
            if self.pool_sizes and i < len(self.pool_sizes):
                self.downsample_factor *= self.pool_sizes[i][0]

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim) -> Tuple[Tensor, Dim]:
        assert self.in_dim in source.dims
        in_spatial_dims = [in_spatial_dim, self.in_dim]
        in_dim = self._dummy_in_dim
        x = _a.expand_dim(source, dim=in_dim)
        for i, conv_layer in enumerate(self.conv_layers):
            x, in_spatial_dims = conv_layer(x, in_spatial_dims=in_spatial_dims)
            in_spatial_dims = list(in_spatial_dims)
            in_dim = conv_layer.out_dim
            x = self.activation(x)
            if self.pool_sizes and i < len(self.pool_sizes):
                x, in_spatial_dims = pool2d(x, in_spatial_dims=in_spatial_dims, pool_size=self.pool_sizes[i], padding="same", mode="max")
                in_spatial_dims = list(in_spatial_dims)
        if in_spatial_dims[-1] != self._final_second_spatial_dim:
            x, in_spatial_dims[-1] = replace_dim(x, out_dim=self._final_second_spatial_dim, in_dim=in_spatial_dims[-1])
        out, _ = _a.merge_dims(x, dims=[self._final_second_spatial_dim, in_dim], out_dim=self.out_dim)
        # layout [B, T, F]
        bt = [d for d in out.dims if d != self.out_dim]
        if out.dims[-1] != self.out_dim or (in_spatial_dims[0] in bt and bt.index(in_spatial_dims[0]) != len(bt) - 1):
            bt = [d for d in bt if d != in_spatial_dims[0]] + [in_spatial_dims[0]]
            out = out.copy_transpose_to_dims(bt + [self.out_dim])
        out.feature_dim = self.out_dim
        return out, in_spatial_dims[0]

    def get_out_spatial_dim(self, in_spatial_dim: Dim) -> Dim:
        """the time dim after subsampling"""
        out_spatial_dim = in_spatial_dim
        for i, conv_layer in enumerate(self.conv_layers):
            (out_spatial_dim,) = make_conv_out_spatial_dims([out_spatial_dim], filter_size=conv_layer.filter_size[0].dimension,
                                                            strides=self._strides2[i][0], padding=conv_layer.padding)
            if self.pool_sizes and i < len(self.pool_sizes):
                (out_spatial_dim,) = make_conv_out_spatial_dims([out_spatial_dim], filter_size=self.pool_sizes[i][0],
                                                                strides=self.pool_sizes[i][0], padding="same")
        return out_spatial_dim


class ConformerEncoderLayer(Module):
    """one Conformer block"""

    def __init__(self, out_dim: Dim = Dim(512, name="conformer-enc-default-out-dim"), *, ff=NotSpecified, ff_dim=NotSpecified,
                 ff_activation=NotSpecified, dropout: float = 0.1, conv_kernel_size: int = 32, conv_norm=NotSpecified,
                 conv_norm_opts: Optional[Dict[str, Any]] = None, num_heads: int = 4, self_att=None,
                 self_att_opts: Optional[Dict[str, Any]] = None, att_dropout: float = 0.1, norm=LayerNorm):
        super().__init__()
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        self.out_dim = out_dim
        self.ffn1 = make_ff(ff=ff, out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, ff_activation=ff_activation)
        self.ffn1_layer_norm = make_norm(norm, out_dim)
        self.ffn2 = make_ff(ff=ff, out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, ff_activation=ff_activation)
        self.ffn2_layer_norm = make_norm(norm, out_dim)
        if conv_norm is NotSpecified or conv_norm is BatchNorm:
            conv_norm_opts = conv_norm_opts.copy() if conv_norm_opts else {}
            conv_norm_opts.setdefault("use_mask", conv_norm_use_mask_default())
            conv_norm = BatchNorm(out_dim, **conv_norm_opts)
        elif isinstance(conv_norm, type):
            conv_norm = conv_norm(out_dim, **(conv_norm_opts or {}))
        elif isinstance(conv_norm, dict):
            conv_norm = build_from_dict(conv_norm, out_dim, **(conv_norm_opts or {}))
        if not callable(conv_norm):
            raise TypeError("%s: unexpected conv_norm type %r" % (self, conv_norm))
        self.conv_block = ConformerConvBlock(out_dim=out_dim, kernel_size=conv_kernel_size, norm=conv_norm)
        self.conv_layer_norm = make_norm(norm, out_dim)
        if self_att is None or isinstance(self_att, (dict, type)):
            opts = dict(in_dim=out_dim, proj_dim=out_dim, key_dim_total=out_dim, value_dim_total=out_dim, num_heads=num_heads, att_dropout=att_dropout)
            if self_att_opts:
                opts.update(self_att_opts)
            if self_att is None:
                self.self_att = RelPosSelfAttention(**opts)
            elif isinstance(self_att, type):
                self.self_att = self_att(**opts)
            else:
                opts = {k: v for k, v in opts.items() if k not in self_att}
                self.self_att = build_from_dict(self_att, **opts)
        else:
            if not callable(self_att):
                raise TypeError("%s: invalid non-callable: self_att %r" % (self, self_att))
            self.self_att = self_att
        self.self_att_layer_norm = make_norm(norm, out_dim)
        self.final_layer_norm = make_norm(norm, out_dim)

    def __call__(self, inp: Tensor, *, spatial_dim: Dim) -> Tensor:
        bc = self.dropout_broadcast and self.out_dim
        x_ffn1 = self.ffn1(self.ffn1_layer_norm(inp))
        x_ffn1_out = 0.5 * dropout(x_ffn1, self.dropout, axis=bc) + inp
        x_mhsa = self.self_att(self.self_att_layer_norm(x_ffn1_out), axis=spatial_dim)
        x_mhsa_out = dropout(x_mhsa, self.dropout, axis=bc) + x_ffn1_out
        x_conv = self.conv_block(self.conv_layer_norm(x_mhsa_out), spatial_dim=spatial_dim)
        x_conv_out = dropout(x_conv, self.dropout, axis=bc) + x_mhsa_out
        x_ffn2 = self.ffn2(self.ffn2_layer_norm(x_conv_out))
        x_ffn2_out = 0.5 * dropout(x_ffn2, self.dropout, axis=bc) + x_conv_out
        return self.final_layer_norm(x_ffn2_out)


class ConformerEncoder(ISeqDownsamplingEncoder):
    """Conformer encoder"""

    def __init__(self, in_dim: Dim, out_dim: Union[Dim, int] = Dim(512, name="conformer-enc-default-out-dim"), *,
                 num_layers: int, input_layer, input_embedding_scale: Optional[float] = None, pos_enc=None,
                 input_dropout: float = 0.1, ff_dim=NotSpecified, ff_activation=NotSpecified, dropout: float = 0.1,
                 conv_kernel_size: int = NotSpecified, conv_norm=NotSpecified, num_heads: int = 4, att_dropout: float = 0.1,
                 encoder_layer=None, encoder_layer_opts: Optional[Dict[str, Any]] = None, sequential=Sequential):
        super().__init__()
        assert isinstance(in_dim, Dim)
        if isinstance(out_dim, int):
            out_dim = Dim(out_dim, name="conformer-enc-out-dim")
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.dropout = dropout
        self.dropout_broadcast = dropout_broadcast_default()
        if callable(input_layer) or input_layer is None:
            pass
        elif isinstance(input_layer, dict):
            input_layer = build_from_dict(input_layer, in_dim)
        else:
            raise TypeError("unexpected input_layer %r" % (input_layer,))
        self.input_layer = input_layer
        in_dim_ = self.input_layer.out_dim if self.input_layer else self.in_dim
        self.input_projection = Linear(in_dim_, self.out_dim, with_bias=False) if in_dim_ != self.out_dim else None
        if input_embedding_scale is None:
            input_embedding_scale = (self.out_dim.dimension ** 0.5) if pos_enc is not None else 1.0
        self.input_embedding_scale = input_embedding_scale
        if pos_enc is None:
            pass
        elif isinstance(pos_enc, dict):
            pos_enc = build_from_dict(pos_enc, feat_dim=self.out_dim)
        elif isinstance(pos_enc, Module):
            pass
        elif isinstance(pos_enc, FunctionType):
            pos_enc = functools.partial(pos_enc, feat_dim=self.out_dim)
        else:
            raise TypeError("unexpected pos_enc type %r" % (pos_enc,))
        self.pos_enc = pos_enc
        self.input_dropout = input_dropout
        encoder_layer = make_encoder_layer(encoder_layer, encoder_layer_opts, owner=self, out_dim=out_dim, ff_dim=ff_dim, ff_activation=ff_activation,
                                           dropout=dropout, conv_kernel_size=conv_kernel_size, conv_norm=conv_norm, num_heads=num_heads, att_dropout=att_dropout)
        self.layers = sequential(_copy.deepcopy(encoder_layer) for _ in range(num_layers))

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim, collected_outputs: Optional[Dict[str, Tensor]] = None) -> Tuple[Tensor, Dim]:
        if self.input_layer and self.input_layer.in_dim in source.dims:
            x, out_spatial_dim = self.input_layer(source, in_spatial_dim=in_spatial_dim)
        else:
            x, out_spatial_dim = source, in_spatial_dim
        if self.input_projection and self.input_projection.in_dim in x.dims:
            x = self.input_projection(x)
        assert self.out_dim in x.dims
        if self.input_embedding_scale != 1.0:
            x = x * self.input_embedding_scale
        if self.pos_enc is not None:
            x = x + self.pos_enc(spatial_dim=out_spatial_dim)
        x = dropout(x, self.input_dropout, axis=self.dropout_broadcast and self.out_dim)
        from .. import packed_mode

        batch_dims = [d for d in x.dims if d not in (out_spatial_dim, self.out_dim)]
        if packed_mode.is_enabled() and len(batch_dims) == 1 and collected_outputs is None:
            # the layers run on the valid frames only: [rows, model] instead of [batch, time, model]
            x = packed_mode.pack_padded_tensor(x, dims=(batch_dims[0], out_spatial_dim))
            x = self.layers(x, spatial_dim=out_spatial_dim)
            return packed_mode.unpack_to_padded(x), out_spatial_dim
        x = self.layers(x, spatial_dim=out_spatial_dim, collected_outputs=collected_outputs)
        return x, out_spatial_dim


def make_encoder_layer(encoder_layer, encoder_layer_opts: Optional[Dict[str, Any]], *, owner=None, **common_opts):
    """
    The prototype layer of an encoder stack from ``None`` (a :class:`ConformerEncoderLayer`), a class, a dict for
    ``build_from_dict`` (the common options fill in what the dict does not name) or a ready module / callable.
    Options that are ``NotSpecified`` are left to the layer's defaults.
    """
    if encoder_layer and not isinstance(encoder_layer, (dict, type)):
        if not callable(encoder_layer):
            raise TypeError("%s: invalid non-callable encoder_layer %r" % (owner, encoder_layer))
        return encoder_layer
    opts = {k: v for k, v in common_opts.items() if v is not NotSpecified}
    if encoder_layer_opts:
        opts.update(encoder_layer_opts)
    if not encoder_layer:
        return ConformerEncoderLayer(**opts)
    if isinstance(encoder_layer, type):
        return encoder_layer(**opts)
    return build_from_dict(encoder_layer, **{k: v for k, v in opts.items() if k not in encoder_layer})


def make_ff(*, out_dim: Dim, ff, ff_dim, ff_activation, dropout: float):
    """the feed-forward part of a Conformer layer from a class / dict / module spec"""
    if ff is NotSpecified:
        ff = ConformerPositionwiseFeedForward
    if isinstance(ff, Module):
        return _copy.deepcopy(ff)
    kw = dict(out_dim=out_dim, ff_dim=ff_dim, dropout=dropout, activation=ff_activation)
    kw = {k: v for k, v in kw.items() if v is not NotSpecified}
    if isinstance(ff, type):
        return ff(**kw)
    if isinstance(ff, dict):
        return build_from_dict(ff, **kw)
    raise TypeError("unexpected ff type %r" % (ff,))


def conv_norm_use_mask_default() -> Optional[bool]:
    """config ``rf_conformer_conv_norm_use_mask``; unmasked statistics up to behavior version 28, then BatchNorm decides"""
    from ...config import get_global_config
    from ...utils.basic import BehaviorVersion

    cfg = get_global_config(raise_exception=False)
    if cfg and cfg.has("rf_conformer_conv_norm_use_mask"):
        return cfg.bool("rf_conformer_conv_norm_use_mask", False)
    if BehaviorVersion.get() >= 29:
        return None
    return False
