"""
HuggingFace Llama (``transformers.models.llama``) -> RF :class:`TransformerDecoder` built with
``RotaryPosCausalSelfAttention``, ``RMSNorm`` and ``FeedForwardGated``
(reference: returnn/frontend/conversions/hf_llama.py:22, :79, :123, :168, :200).

Layout differences handled here:

* torch Linear weights are (out, in), RF's (in, out);
* ``gate_proj`` and ``up_proj`` become the two halves of ``FeedForwardGated.linear_ff`` (gate first);
* RF keeps q, k, v in ONE projection whose output is ordered (head, [q | k | v]);
* HF rotates the feature pairs (i, i + D/2) of each head, RF the pairs (2i, 2i + 1): the q and k columns of each head are
  permuted so that HF's feature ``i`` lands at ``2i`` and ``i + D/2`` at ``2i + 1``. Scores are unchanged, since q and k get
  the same permutation.

The modules are addressed by attribute names only, so any model with Llama's module tree can be imported.
"""

from __future__ import annotations
import torch
from ..attention import RotaryPosCausalSelfAttention
from ..normalization import RMSNorm
from ..decoder.transformer import TransformerDecoder, TransformerDecoderLayer, FeedForwardGated
from ._common import assign, check_same_num_params

__all__ = [
    "import_params_hf_llama_to_rf_transformer_decoder",
    "import_params_hf_llama_decoder_layer_to_rf",
    "import_params_hf_llama_mlp_to_rf_feed_forward_gated",
    "import_params_hf_llama_rms_norm_to_rf",
    "import_params_hf_llama_att_to_rf_rotary_att",
]


def import_params_hf_llama_to_rf_transformer_decoder(model_hf, model_rf: TransformerDecoder):
    """``LlamaModel`` (no output layer: ``model_rf.logits`` is left alone) or ``LlamaForCausalLM``"""
    lm_head = getattr(model_hf, "lm_head", None)
    exclude = []
    core = model_hf.model if lm_head is not None else model_hf
    if lm_head is None:
        exclude.append(model_rf.logits.weight)
    if len(core.layers) != len(model_rf.layers):
        raise ValueError("the source has %i layers, the RF decoder %i" % (len(core.layers), len(model_rf.layers)))
    for layer_hf, layer_rf in zip(core.layers, model_rf.layers):
        import_params_hf_llama_decoder_layer_to_rf(layer_hf, layer_rf)
    assign(model_rf.input_embedding.weight, core.embed_tokens.weight, what="input_embedding.weight")
    if not isinstance(model_rf.final_layer_norm, RMSNorm):
        raise TypeError("final_layer_norm must be an RMSNorm, got %r" % (model_rf.final_layer_norm,))
    import_params_hf_llama_rms_norm_to_rf(core.norm, model_rf.final_layer_norm)
    if lm_head is not None:
        if lm_head.bias is not None or model_rf.logits.with_bias:
            raise NotImplementedError("an output layer with bias")
        tied = lm_head.weight is core.embed_tokens.weight or lm_head.weight.data_ptr() == core.embed_tokens.weight.data_ptr()
        if model_rf.logits.weight is model_rf.input_embedding.weight:
            if not tied and not torch.equal(lm_head.weight, core.embed_tokens.weight):
                raise ValueError("the RF decoder shares embedding and output weights, the source does not")
        else:
            assign(model_rf.logits.weight, lm_head.weight.T, what="logits.weight")
    check_same_num_params(model_hf, model_rf, what="Llama", exclude_rf=exclude)


def import_params_hf_llama_decoder_layer_to_rf(model_hf, model_rf: TransformerDecoderLayer):
    """``LlamaDecoderLayer``"""
    if not isinstance(model_rf.ff, FeedForwardGated):
        raise TypeError("the layer's ff must be a FeedForwardGated, got %r" % (model_rf.ff,))
    if not isinstance(model_rf.self_att, RotaryPosCausalSelfAttention):
        raise TypeError("the layer's self_att must be a RotaryPosCausalSelfAttention, got %r" % (model_rf.self_att,))
    import_params_hf_llama_mlp_to_rf_feed_forward_gated(model_hf.mlp, model_rf.ff)
    import_params_hf_llama_att_to_rf_rotary_att(model_hf.self_attn, model_rf.self_att)
    for norm_hf, norm_rf, name in ((model_hf.input_layernorm, model_rf.self_att_layer_norm, "self_att_layer_norm"),
                                   (model_hf.post_attention_layernorm, model_rf.ff_layer_norm, "ff_layer_norm")):
        if not isinstance(norm_rf, RMSNorm):
            raise TypeError("%s must be an RMSNorm, got %r" % (name, norm_rf))
        import_params_hf_llama_rms_norm_to_rf(norm_hf, norm_rf)
    check_same_num_params(model_hf, model_rf, what="Llama decoder layer")


def import_params_hf_llama_mlp_to_rf_feed_forward_gated(model_hf, model_rf: FeedForwardGated):
    """``LlamaMLP``: down(act(gate(x)) * up(x))"""
    for name in ("gate_proj", "up_proj", "down_proj"):
        if getattr(model_hf, name).bias is not None:
            raise NotImplementedError("Llama MLP with bias (%s)" % name)
    w = torch.cat((model_hf.gate_proj.weight.T, model_hf.up_proj.weight.T), dim=1)  # (in, 2 * ff)
    assign(model_rf.linear_ff.weight, w, what="ff.linear_ff.weight")
    assign(model_rf.linear_out.weight, model_hf.down_proj.weight.T, what="ff.linear_out.weight")
    check_same_num_params(model_hf, model_rf, what="Llama MLP")


def import_params_hf_llama_rms_norm_to_rf(model_hf, model_rf: RMSNorm):
    """``LlamaRMSNorm``"""
    assign(model_rf.scale, model_hf.weight, what="RMSNorm.scale")
    check_same_num_params(model_hf, model_rf, what="Llama RMSNorm")


def _rope_pairs_half_to_interleaved(w: torch.Tensor) -> torch.Tensor:
    """(in, heads, D) with rotation pairs (i, i + D/2) -> pairs (2i, 2i + 1)"""
    d_in, nh, hd = w.shape
    return w.reshape(d_in, nh, 2, hd // 2).transpose(-1, -2).reshape(d_in, nh, hd)


def import_params_hf_llama_att_to_rf_rotary_att(model_hf, model_rf: RotaryPosCausalSelfAttention):
    """``LlamaAttention`` with as many key/value heads as query heads"""
    dim = model_rf.in_dim.dimension
    nh = model_rf.num_heads.dimension
    hd = model_rf.key_dim_per_head.dimension
    if model_hf.q_proj.weight.shape != (nh * hd, dim) or model_hf.k_proj.weight.shape != (nh * hd, dim):
        raise ValueError("attention shapes differ: q %s, k %s in the source; RF has %i heads of %i over %i inputs (grouped-query attention is not covered)"
                         % (tuple(model_hf.q_proj.weight.shape), tuple(model_hf.k_proj.weight.shape), nh, hd, dim))
    if model_hf.q_proj.bias is not None:
        raise NotImplementedError("Llama attention with bias")
    q = _rope_pairs_half_to_interleaved(model_hf.q_proj.weight.T.reshape(dim, nh, hd))
    k = _rope_pairs_half_to_interleaved(model_hf.k_proj.weight.T.reshape(dim, nh, hd))
    v = model_hf.v_proj.weight.T.reshape(dim, nh, -1)
    assign(model_rf.qkv.weight, torch.cat([q, k, v], dim=2).reshape(dim, -1), what="self_att.qkv.weight")
    assign(model_rf.proj.weight, model_hf.o_proj.weight.T, what="self_att.proj.weight")
    check_same_num_params(model_hf, model_rf, what="Llama attention")
