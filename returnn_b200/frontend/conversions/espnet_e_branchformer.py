"""
ESPnet E-Branchformer encoder layer (``espnet2.asr.encoder.e_branchformer_encoder.EBranchformerEncoderLayer``) ->
:class:`returnn_b200.frontend.encoder.e_branchformer.EBranchformerLayer`
(reference: returnn/frontend/conversions/espnet_e_branchformer.py:23, :71, :80, :137, :164).

The source modules are addressed by attribute names only (``feed_forward.w_1``, ``attn.linear_q``, ``cgmlp.csgu.conv`` ...),
so ESPnet itself is not needed to run the import, and any module tree with these names works.

Layout differences handled here:

* q, k, v projections are separate in ESPnet and one projection ordered (head, [q | k | v]) in RF;
* relative positions: ESPnet's encoding of distance p is interleaved ``(sin(p w_i), cos(p w_i))`` and its score uses
  p = query - key; RF's is ``[sin | cos]`` of p' = key - query. With sin odd and cos even, ``linear_pos`` gives the same
  result when its sin rows are negated and the rows are de-interleaved;
* cgMLP: ESPnet gates the SECOND half of the projected features with the first (``x_r, x_g = chunk(2)``), RF normalises and
  convolves the FIRST half, so the two halves of ``channel_proj1`` are swapped.
"""

from __future__ import annotations
import torch
from ..attention import SelfAttention, RelPosSelfAttention
from ..decoder.transformer import FeedForward
from ..encoder.e_branchformer import EBranchformerLayer, FeedForwardConvGated
from ._common import assign, check_same_num_params
from .torch_nn import import_params_torch_conv1d_to_rf, import_params_torch_layer_norm_to_rf, import_params_torch_linear_to_rf

__all__ = [
    "import_params_espnet_e_branchformer_layer_to_rf",
    "import_params_espnet_positionwise_feed_forward_to_rf",
    "import_params_espnet_multi_headed_attention_to_rf",
    "import_params_espnet_convolutional_gating_mlp_to_rf",
]


def import_params_espnet_e_branchformer_layer_to_rf(model_espnet, model_rf: EBranchformerLayer):
    """one encoder layer"""
    if not isinstance(model_rf, EBranchformerLayer):
        raise TypeError("expected an EBranchformerLayer, got %r" % (model_rf,))
    import_params_espnet_positionwise_feed_forward_to_rf(model_espnet.feed_forward_macaron, model_rf.ffn1)
    import_params_espnet_positionwise_feed_forward_to_rf(model_espnet.feed_forward, model_rf.ffn2)
    for src, dst in ((model_espnet.norm_ff_macaron, model_rf.ffn1_layer_norm), (model_espnet.norm_ff, model_rf.ffn2_layer_norm),
                     (model_espnet.norm_mha, model_rf.self_att_layer_norm), (model_espnet.norm_mlp, model_rf.cgmlp_layer_norm),
                     (model_espnet.norm_final, model_rf.final_layer_norm)):
        import_params_torch_layer_norm_to_rf(src, dst)
    import_params_espnet_multi_headed_attention_to_rf(model_espnet.attn, model_rf.self_att)
    import_params_espnet_convolutional_gating_mlp_to_rf(model_espnet.cgmlp, model_rf.cgmlp)
    import_params_torch_conv1d_to_rf(model_espnet.depthwise_conv_fusion, model_rf.merge.depthwise_conv_fusion)
    import_params_torch_linear_to_rf(model_espnet.merge_proj, model_rf.merge.merge_proj)
    check_same_num_params(model_espnet, model_rf, what="E-Branchformer layer")


def import_params_espnet_positionwise_feed_forward_to_rf(model_espnet, model_rf: FeedForward):
    """``PositionwiseFeedForward``: w_2(dropout(act(w_1(x))))"""
    import_params_torch_linear_to_rf(model_espnet.w_1, model_rf.linear_ff)
    import_params_torch_linear_to_rf(model_espnet.w_2, model_rf.linear_out)


def reorder_rel_pos_emb_espnet_to_rf(x: torch.Tensor, *, dim: int = -1) -> torch.Tensor:
    """along ``dim``: interleaved (sin, cos) of distance p -> [sin | cos] of distance -p"""
    x = x.movedim(dim, -1)
    *lead, d = x.shape
    x = x.reshape(*lead, d // 2, 2)
    x = torch.stack((-x[..., 0], x[..., 1]), dim=-2)  # [..., 2, D/2]: negated sin rows, then cos rows
    return x.reshape(*lead, d).movedim(-1, dim)


def import_params_espnet_multi_headed_attention_to_rf(model_espnet, model_rf):
    """``MultiHeadedAttention`` -> SelfAttention, ``RelPositionMultiHeadedAttention`` (new style) -> RelPosSelfAttention"""
    if not isinstance(model_rf, (SelfAttention, RelPosSelfAttention)):
        raise TypeError("expected SelfAttention or RelPosSelfAttention, got %r" % (model_rf,))
    nh, hd = model_espnet.h, model_espnet.d_k
    if (nh, hd) != (model_rf.num_heads.dimension, model_rf.key_dim_per_head.dimension):
        raise ValueError("heads x dim: source %i x %i, RF %i x %i" % (nh, hd, model_rf.num_heads.dimension, model_rf.key_dim_per_head.dimension))
    dim = nh * hd
    ws = [getattr(model_espnet, n).weight.T.reshape(dim, nh, hd) for n in ("linear_q", "linear_k", "linear_v")]
    bs = [getattr(model_espnet, n).bias.reshape(nh, hd) for n in ("linear_q", "linear_k", "linear_v")]
    assign(model_rf.qkv.weight, torch.cat(ws, dim=2).reshape(dim, 3 * dim), what="self_att.qkv.weight")
    assign(model_rf.qkv.bias, torch.cat(bs, dim=1).reshape(3 * dim), what="self_att.qkv.bias")
    import_params_torch_linear_to_rf(model_espnet.linear_out, model_rf.proj)
    has_pos = hasattr(model_espnet, "linear_pos")
    if has_pos != isinstance(model_rf, RelPosSelfAttention):
        raise TypeError("relative positions on one side only (source: %s, RF: %s)" % (has_pos, type(model_rf).__name__))
    if has_pos:
        if model_rf.linear_pos is None or model_rf.pos_bias_u is None or model_rf.pos_bias_v is None:
            raise ValueError("the RF attention needs with_linear_pos=True and with_pos_bias=True")
        assign(model_rf.linear_pos.weight, reorder_rel_pos_emb_espnet_to_rf(model_espnet.linear_pos.weight.T, dim=0), what="self_att.linear_pos.weight")
        assign(model_rf.pos_bias_u, model_espnet.pos_bias_u, what="self_att.pos_bias_u")
        assign(model_rf.pos_bias_v, model_espnet.pos_bias_v, what="self_att.pos_bias_v")
    check_same_num_params(model_espnet, model_rf, what="attention")


def import_params_espnet_convolutional_gating_mlp_to_rf(model_espnet, model_rf: FeedForwardConvGated):
    """``ConvolutionalGatingMLP`` with the default CSGU (no ``linear`` after the conv)"""
    if not isinstance(model_rf, FeedForwardConvGated):
        raise TypeError("expected FeedForwardConvGated, got %r" % (model_rf,))
    if getattr(model_espnet.csgu, "linear", None) is not None:
        raise NotImplementedError("CSGU with use_linear_after_conv")
    proj1 = model_espnet.channel_proj1[0]
    f = model_rf.ff_dim.dimension
    w = proj1.weight.T  # (in, 2F): ESPnet's first half is the pass-through part, its second half is gated
    assign(model_rf.linear_ff.weight, torch.cat((w[:, f:], w[:, :f]), dim=1), what="cgmlp.linear_ff.weight")
    if model_rf.linear_ff.with_bias:
        assign(model_rf.linear_ff.bias, torch.cat((proj1.bias[f:], proj1.bias[:f])), what="cgmlp.linear_ff.bias")
    import_params_torch_linear_to_rf(model_espnet.channel_proj2, model_rf.linear_out)
    import_params_torch_layer_norm_to_rf(model_espnet.csgu.norm, model_rf.norm)
    import_params_torch_conv1d_to_rf(model_espnet.csgu.conv, model_rf.conv)
    check_same_num_params(model_espnet, model_rf, what="cgMLP")
