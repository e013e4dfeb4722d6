"""
Fused execution path of the Conformer encoder on packed rows (B200).

Input: padded features ``[B, T, F]`` + host lengths. The conv2d subsampling frontend runs on the padded batch; from
there on only the valid frames exist, as rows ``[N, D]`` with ``cu_seqlens``. Every block is a chain of the ops in
:mod:`returnn_b200.ops` (LayerNorm, GEMM with bias/activation epilogue, relative-position attention over the sequence
offsets, GLU + depthwise conv + masked BatchNorm + SiLU, dropout), each with its hand-written backward, so one step is a
few hundred launches that a CUDA graph replays.

The parameters are those of :class:`returnn_b200.frontend.encoder.conformer.ConformerEncoder` (same module tree, same
checkpoint keys); this file only changes how the forward pass is executed.
"""

from __future__ import annotations
from typing import Dict, Optional, Tuple
import math
import torch
import torch.nn.functional as F
from .packing import PackInfo
from ..ops import layer_norm as _ln
from ..ops import linear as _lin
from ..ops import conv_module as _cm
from ..ops import attention_packed as _att
from ..ops import elementwise as _ew


class _Weights:
    """bf16 views of the fp32 master weights, cast once per step (the cast is differentiable)"""

    def __init__(self, dtype: torch.dtype):
        self.dtype = dtype
        self._cache: Dict[int, torch.Tensor] = {}

    def __call__(self, p) -> Optional[torch.Tensor]:
        if p is None:
            return None
        raw = p.raw_tensor if hasattr(p, "raw_tensor") else p
        key = id(raw)
        t = self._cache.get(key)
        if t is None:
            t = raw if raw.dtype == self.dtype else raw.to(self.dtype)
            self._cache[key] = t
        return t


def _dropout(x: torch.Tensor, p: float, training: bool) -> torch.Tensor:
    if not training or not p:
        return x
    if x.is_cuda and x.dtype == torch.bfloat16 and _ew.available():
        return _ew.dropout(x, p)
    return F.dropout(x, p, training=True)


def frontend_subsample(enc, feats: torch.Tensor, lens_host: torch.Tensor, W: _Weights) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    conv2d subsampling stack on the padded batch.

    :param feats: [B, T, F]
    :return: [B, T', F'*C] and the new host lengths
    """
    from ..frontend.conv import _same_pads

    from .packing import host_to_device

    il = enc.input_layer
    B, T, Fdim = feats.shape
    # lengths after every stage, computed on the host and sent in one asynchronous copy
    stage_lens = [lens_host.clone().to(torch.int64)]
    for i, conv in enumerate(il.conv_layers):
        fs = tuple(d.dimension for d in conv.filter_size)
        st = il._strides2[i]
        lens = stage_lens[-1]
        if conv.padding == "same":
            lens = -(-lens // st[0])
        else:
            lens = torch.clamp(-(-(lens - fs[0] + 1) // st[0]), min=0)
        if il.pool_sizes and i < len(il.pool_sizes):
            lens = -(-lens // il.pool_sizes[i][0])
        stage_lens.append(lens)
    lens_dev = host_to_device(torch.stack(stage_lens).to(torch.int32), feats.device)
    mask = torch.arange(T, device=feats.device)[None, :] < lens_dev[0][:, None]
    x = (feats * mask.unsqueeze(-1).to(feats.dtype)).unsqueeze(1)  # [B,1,T,F]
    x = x.contiguous(memory_format=torch.channels_last)
    for i, conv in enumerate(il.conv_layers):
        fs = tuple(d.dimension for d in conv.filter_size)
        st = il._strides2[i]
        w = W(conv.filter)
        b = W(conv.bias)
        if conv.padding == "same":
            pads = _same_pads(x.shape[2:], fs, st)
            if any(pads):
                x = F.pad(x, pads)
        x = F.conv2d(x, w, b, stride=st)
        x = torch.relu(x)
        if il.pool_sizes and i < len(il.pool_sizes):
            ps = il.pool_sizes[i]
            pads = _same_pads(x.shape[2:], ps, ps)
            if any(pads):
                x = F.pad(x, pads, value=float("-inf"))
            x = F.max_pool2d(x, kernel_size=ps, stride=ps)
        # frames past each sequence's end must be zero for the next conv
        Tn = x.shape[2]
        m = (torch.arange(Tn, device=x.device)[None, :] < lens_dev[i + 1][:, None]).to(x.dtype)
        x = x * m[:, None, :, None]
    lens = stage_lens[-1]
    Bc, C, Tn, Fn = x.shape
    out = x.permute(0, 2, 3, 1).reshape(Bc, Tn, Fn * C)
    return out, lens.to(torch.int32)


def _frontend_native(enc, feats: torch.Tensor, lens_host: torch.Tensor):
    """conv subsampling through the implicit-GEMM kernels; (None, None) if the configuration is not covered"""
    from ..ops import frontend_native as _fe
    from .packing import host_to_device

    il = enc.input_layer
    if not _fe.available(feats):
        return None, None
    convs = list(il.conv_layers)
    chans = tuple(c.out_dim.dimension for c in convs)
    fsz = [tuple(d.dimension for d in c.filter_size) for c in convs]
    strides = [tuple(s) for s in il._strides2]
    if any(c.padding != "same" for c in convs) or not _fe.supports(feats.shape[-1], chans, fsz, strides, il.pool_sizes):
        return None, None
    if convs[0].in_dim.dimension != 1:
        return None, None
    lens0 = lens_host.clone().to(torch.int64)
    lens1 = -(-lens0 // strides[1][0])
    lens2 = -(-lens1 // strides[2][0])
    # the padded lengths of the intermediate tensors follow the padded input length, like the torch path
    pack = PackInfo(lens2.to(torch.int32), feats.device)
    lens_dev = host_to_device(torch.stack([lens0, lens1, lens2]).to(torch.int32), feats.device)
    params = [(c.filter.raw_tensor, c.bias.raw_tensor if c.bias is not None else None) for c in convs]
    x = _fe.conv_subsample_packed(feats.to(torch.bfloat16), lens_dev, pack, params, (strides[1][0], strides[2][0]))
    return x, pack


def ffn_block(x, layer_norm, ff, W, p_drop, training, eps):
    """0.5 * dropout(FFN(LN(x))) + x"""
    h = _ln.layer_norm(x, W(layer_norm.scale), W(layer_norm.bias), eps)
    h = _lin.linear(h, W(ff.linear_ff.weight), W(ff.linear_ff.bias), "silu")
    h = _dropout(h, ff.dropout, training)
    h = _lin.linear(h, W(ff.linear_out.weight), W(ff.linear_out.bias))
    h = _dropout(h, p_drop, training)
    return x + 0.5 * h


def mhsa_block(x, layer, pack: PackInfo, pos_proj, W, p_drop, training, eps):
    """dropout(MHSA(LN(x))) + x"""
    sa = layer.self_att
    H = sa.num_heads.dimension
    Dk = sa.key_dim_per_head.dimension
    h = _ln.layer_norm(x, W(layer.self_att_layer_norm.scale), W(layer.self_att_layer_norm.bias), eps)
    qkv = _lin.linear(h, W(sa.qkv.weight), W(sa.qkv.bias))  # [N, H*3*Dk] grouped per head as (q,k,v)
    att = _att.rel_pos_attention_packed(qkv, pos_proj, W(sa.pos_bias_u), W(sa.pos_bias_v), pack, num_heads=H, head_dim=Dk,
                                        scale=Dk ** -0.5, dropout_p=sa.att_dropout if training else 0.0)  # [N, H*Dk]
    out = _lin.linear(att, W(sa.proj.weight), W(sa.proj.bias))
    return x + _dropout(out, p_drop, training)


def conv_block(x, layer, pack: PackInfo, W, p_drop, training, eps):
    """dropout(ConvModule(LN(x))) + x"""
    cb = layer.conv_block
    h = _ln.layer_norm(x, W(layer.conv_layer_norm.scale), W(layer.conv_layer_norm.bias), eps)
    h = _lin.linear(h, W(cb.positionwise_conv1.weight), W(cb.positionwise_conv1.bias))  # [N, 2D]
    bn = cb.norm
    # small fp32 parameters go in as they are: the kernels read fp32 filter / BatchNorm parameters
    h = _cm.glu_dwconv_bn_silu(h, cb.depthwise_conv.filter.raw_tensor, cb.depthwise_conv.bias.raw_tensor if cb.depthwise_conv.bias is not None else None,
                               bn, pack, training=training)
    h = _lin.linear(h, W(cb.positionwise_conv2.weight), W(cb.positionwise_conv2.bias))
    return x + _dropout(h, p_drop, training)


def pos_projection(enc, max_len: int, device, dtype, W) -> Optional[torch.Tensor]:
    """
    projected relative positional embeddings of the first layer's geometry: per layer ``linear_pos(sinusoid)``
    is computed by the caller per layer (weights differ); this returns the raw sinusoid ``[2*max_len-1, D]``.
    """
    D = enc.out_dim.dimension
    idx = torch.arange(-(max_len - 1), max_len, device=device, dtype=torch.float32)
    # the frequency spacing of rf.relative_positional_encoding, 1e4 ** (-2i / D) (returnn/frontend/attention.py:1189; the absolute
    # sinusoidal encoding spaces its frequencies differently); tests/test_native_encoder_gpu.py checks the whole encoder against an
    # fp32 run of the RF module
    div = torch.exp(torch.arange(D // 2, device=device, dtype=torch.float32) * -(2.0 * math.log(1e4) / D))
    arg = idx[:, None] * div[None, :]
    return torch.cat([torch.sin(arg), torch.sin(arg + math.pi / 2.0)], dim=-1).to(dtype)


def arena_linear(x, weight, bias, act, arena, W):
    """linear layer through the arena path (bf16 weight copy, gradients accumulated in place) when possible"""
    from ..ops import gemm as _gemm

    if arena is not None:
        y = _gemm.linear_arena(x, weight, bias, act, arena)
        if y is not None:
            return y
    return _lin.linear(x, W(weight), W(bias) if bias is not None else None, act)


def _att_supports(plan, pack: PackInfo) -> bool:
    from ..ops import attention_native as _an

    return _an.supports_packed(plan.H, plan.Dh, pack.max_len) and plan.D % 64 == 0 and plan.H * plan.Dh == plan.D and 1 <= plan.conv_k <= 64


def supports_fused(enc) -> bool:
    """whether the encoder is in the standard configuration that the fused path implements"""
    from ..frontend.encoder.conformer import ConformerEncoderLayer, ConformerConvSubsample, ConformerPositionwiseFeedForward
    from ..frontend.attention import RelPosSelfAttention
    from ..frontend.normalization import LayerNorm, BatchNorm
    from ..frontend import math_ as _m

    if not isinstance(enc.input_layer, ConformerConvSubsample) or enc.pos_enc is not None or enc.input_projection is None:
        return False
    # this path works on valid frames only: it computes what the RF modules compute when convolutions mask their padded input
    # (default from behavior version 23) and the BatchNorm statistics leave the padded frames out (use_mask)
    from ..frontend.dims import use_mask_default

    if not use_mask_default(default=True, default_false_for_behavior_version_up_to=22):
        return False
    if enc.input_layer.activation is not _m.relu:
        return False
    for layer in enc.layers:
        if type(layer) is not ConformerEncoderLayer and not isinstance(layer, ConformerEncoderLayer):
            return False
        sa = layer.self_att
        if not isinstance(sa, RelPosSelfAttention) or sa.linear_pos is None or sa.learned_pos_emb is not None or not sa.separate_pos_emb_per_head:
            return False
        if sa.pos_emb_dropout or sa.att_dropout_broadcast:
            return False
        if not isinstance(layer.conv_block.norm, BatchNorm) or not isinstance(layer.ffn1_layer_norm, LayerNorm):
            return False
        bn_mask = layer.conv_block.norm.use_mask
        if bn_mask is None:  # BatchNorm's own default: config rf_batch_norm_use_mask, else unmasked
            from ..config import get_global_config

            cfg = get_global_config(raise_exception=False)
            bn_mask = cfg.bool("rf_batch_norm_use_mask", False) if cfg else False
        if not bn_mask:
            return False
        if not isinstance(layer.ffn1, ConformerPositionwiseFeedForward) or layer.ffn1.activation is not _m.swish:
            return False
        if layer.dropout_broadcast:
            return False
    return True


def encode_packed(enc, feats: torch.Tensor, lens_host: torch.Tensor, *, training: bool, compute_dtype=torch.bfloat16,
                  collected: Optional[Dict[str, torch.Tensor]] = None) -> Tuple[torch.Tensor, PackInfo]:
    """
    :param enc: ConformerEncoder (RF module)
    :param feats: [B, T, F] on the device
    :param lens_host: int32 [B] on the host
    :return: rows [N, D] in compute_dtype, their PackInfo
    """
    from . import conformer_native as _native

    W = _Weights(compute_dtype)
    x = None
    if compute_dtype == torch.bfloat16 and feats.is_cuda:
        x, pack = _frontend_native(enc, feats, lens_host)
    if x is None:
        x_pad, lens2 = frontend_subsample(enc, feats.to(compute_dtype), lens_host, W)
        pack = PackInfo(lens2, feats.device, padded_len=x_pad.shape[1])
        x = pack.pack(x_pad)
    plan = None
    if training and torch.is_grad_enabled() and compute_dtype == torch.bfloat16 and collected is None and x.is_cuda:
        plan = _native.get_plan(enc)
    x = arena_linear(x, enc.input_projection.weight.raw_tensor, None, None, plan.arena if plan is not None else None, W)
    if enc.input_embedding_scale != 1.0:
        x = x * enc.input_embedding_scale
    x = _dropout(x, enc.input_dropout, training)
    sinus = pos_projection(enc, pack.max_len, feats.device, compute_dtype, W)
    if plan is not None and _att_supports(plan, pack):
        # the whole layer stack as one native call per pass
        x = _native.encoder_stack(x, sinus, plan, pack)
        return x, pack
    for name, layer in enc.layers._get_modules().items():
        eps = layer.ffn1_layer_norm.eps
        p = layer.dropout
        x = ffn_block(x, layer.ffn1_layer_norm, layer.ffn1, W, p, training, eps)
        pos_proj = _lin.linear(sinus, W(layer.self_att.linear_pos.weight), None)  # [2L-1, H*Dk]
        x = mhsa_block(x, layer, pack, pos_proj, W, p, training, eps)
        x = conv_block(x, layer, pack, W, p, training, eps)
        x = ffn_block(x, layer.ffn2_layer_norm, layer.ffn2, W, p, training, eps)
        x = _ln.layer_norm(x, W(layer.final_layer_norm.scale), W(layer.final_layer_norm.bias), eps)
        if collected is not None:
            collected[name] = x
    return x, pack
