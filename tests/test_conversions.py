"""
Parameter import from other toolkits (returnn_b200/frontend/conversions): after the import the RF module computes what the source
module computes. HuggingFace Llama is checked against ``transformers`` itself; the ESPnet E-Branchformer layer against a torch
re-statement of ESPnet's layer written here from its published structure (ESPnet is not installed).
"""

import math
import numpy
import pytest
import torch

import returnn_b200.frontend as rf
from returnn_b200.tensor import Tensor, Dim, batch_dim


def _time_dim(lens):
    batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(len(lens), dtype=torch.int32))
    d = Dim(None, name="time")
    d.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor(lens, dtype=torch.int32))
    return d


def test_torch_nn_importers():
    from returnn_b200.frontend.conversions.torch_nn import (
        import_params_torch_linear_to_rf, import_params_torch_conv1d_to_rf, import_params_torch_layer_norm_to_rf)

    torch.manual_seed(0)
    i, o = Dim(5, name="in"), Dim(7, name="out")
    time = _time_dim([9, 6])
    x_raw = torch.randn(2, 9, 5)
    x = Tensor("x", dims=[batch_dim, time, i], dtype="float32", raw_tensor=x_raw)
    lin_pt, lin_rf = torch.nn.Linear(5, 7), rf.Linear(i, o)
    import_params_torch_linear_to_rf(lin_pt, lin_rf)
    assert torch.allclose(lin_rf(x).copy_transpose([batch_dim, time, o]).raw_tensor, lin_pt(x_raw), atol=1e-6)
    ln_pt, ln_rf = torch.nn.LayerNorm(5, eps=1e-6), rf.LayerNorm(i)
    with torch.no_grad():
        ln_pt.weight.uniform_(0.5, 1.5)
        ln_pt.bias.uniform_(-0.5, 0.5)
    import_params_torch_layer_norm_to_rf(ln_pt, ln_rf)
    assert torch.allclose(ln_rf(x).copy_transpose([batch_dim, time, i]).raw_tensor, ln_pt(x_raw), atol=1e-5)
    conv_pt, conv_rf = torch.nn.Conv1d(5, 7, 3, padding=1), rf.Conv1d(i, o, filter_size=3, padding="same")
    import_params_torch_conv1d_to_rf(conv_pt, conv_rf)
    y, _ = conv_rf(x, in_spatial_dim=time)
    ref = conv_pt(x_raw.transpose(1, 2)).transpose(1, 2)
    assert torch.allclose(y.copy_transpose([batch_dim, time, o]).raw_tensor[0], ref[0], atol=1e-5)  # the full-length sequence
    with pytest.raises(ValueError):
        import_params_torch_linear_to_rf(torch.nn.Linear(5, 7, bias=False), lin_rf)
    with pytest.raises(ValueError):
        import_params_torch_linear_to_rf(torch.nn.Linear(4, 7), lin_rf)


def test_hf_llama_import_gives_the_same_logits():
    from transformers.models.llama.modeling_llama import LlamaForCausalLM, LlamaConfig
    from returnn_b200.frontend.decoder.transformer import TransformerDecoder, FeedForwardGated
    from returnn_b200.frontend.conversions.hf_llama import import_params_hf_llama_to_rf_transformer_decoder

    torch.manual_seed(1)
    cfg = LlamaConfig(vocab_size=17, hidden_size=16, intermediate_size=24, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                      max_position_embeddings=64, rms_norm_eps=1e-6, initializer_range=0.4, tie_word_embeddings=False, attention_dropout=0.0)
    hf = LlamaForCausalLM(cfg).eval()
    vocab, model = Dim(17, name="vocab"), Dim(16, name="model")
    dec = TransformerDecoder(
        None, vocab, model, num_layers=2, num_heads=4, pos_enc=None, norm=rf.build_dict(rf.RMSNorm, eps=1e-6), ff=rf.build_dict(FeedForwardGated, ff_dim=24),
        layer_opts=dict(self_att=rf.build_dict(rf.RotaryPosCausalSelfAttention, with_bias=False)), share_embedding=False, input_embedding_scale=1.0,
        dropout=0.0, att_dropout=0.0)
    import_params_hf_llama_to_rf_transformer_decoder(hf, dec)
    rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)
    lens = [11, 7]
    time = _time_dim(lens)
    ids = torch.randint(0, 17, (2, 11))
    x = Tensor("x", dims=[batch_dim, time], dtype="int64", sparse_dim=vocab, raw_tensor=ids)
    with torch.no_grad():
        logits, _ = dec(x, spatial_dim=time, state=dec.default_initial_state(batch_dims=[batch_dim]))
        ref = hf(input_ids=ids).logits
    got = logits.copy_transpose([batch_dim, time, vocab]).raw_tensor
    for b, n in enumerate(lens):  # causal: the padded tail of the shorter sequence does not reach its real positions
        assert torch.allclose(got[b, :n], ref[b, :n], atol=2e-5), float((got[b, :n] - ref[b, :n]).abs().max())
    # the core model without output layer: logits stay as they were
    dec2 = TransformerDecoder(
        None, vocab, model, num_layers=2, num_heads=4, pos_enc=None, norm=rf.build_dict(rf.RMSNorm, eps=1e-6), ff=rf.build_dict(FeedForwardGated, ff_dim=24),
        layer_opts=dict(self_att=rf.build_dict(rf.RotaryPosCausalSelfAttention, with_bias=False)), share_embedding=False, dropout=0.0, att_dropout=0.0)
    before = dec2.logits.weight.raw_tensor.clone()
    import_params_hf_llama_to_rf_transformer_decoder(hf.model, dec2)
    assert torch.equal(dec2.logits.weight.raw_tensor, before)
    assert torch.equal(dec2.layers[1].ff.linear_out.weight.raw_tensor, hf.model.layers[1].mlp.down_proj.weight.T)


# ---- ESPnet's E-Branchformer layer, restated in torch (module and attribute names as in ESPnet) -----------------------------------------
class _EspnetFF(torch.nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.w_1, self.w_2 = torch.nn.Linear(d, h), torch.nn.Linear(h, d)

    def forward(self, x):
        return self.w_2(torch.nn.functional.silu(self.w_1(x)))


class _EspnetRelPosMHA(torch.nn.Module):
    """RelPositionMultiHeadedAttention (new style): pos_emb runs over distances T-1 .. -(T-1)"""

    def __init__(self, h, d):
        super().__init__()
        self.h, self.d_k = h, d // h
        self.linear_q, self.linear_k, self.linear_v, self.linear_out = (torch.nn.Linear(d, d) for _ in range(4))
        self.linear_pos = torch.nn.Linear(d, d, bias=False)
        self.pos_bias_u = torch.nn.Parameter(torch.randn(h, self.d_k) * 0.3)
        self.pos_bias_v = torch.nn.Parameter(torch.randn(h, self.d_k) * 0.3)

    @staticmethod
    def rel_shift(x):
        b, h, t, n = x.shape
        x = torch.cat([torch.zeros(b, h, t, 1), x], dim=-1).view(b, h, n + 1, t)
        return x[:, :, 1:].view_as(x[:, :, 1:].reshape(b, h, t, n))[:, :, :, : n // 2 + 1]

    def forward(self, x, pos_emb, mask):
        b, t, _ = x.shape
        q = self.linear_q(x).view(b, t, self.h, self.d_k)
        k = self.linear_k(x).view(b, t, self.h, self.d_k).transpose(1, 2)
        v = self.linear_v(x).view(b, t, self.h, self.d_k).transpose(1, 2)
        p = self.linear_pos(pos_emb).view(1, -1, self.h, self.d_k).transpose(1, 2)
        ac = torch.matmul((q + self.pos_bias_u).transpose(1, 2), k.transpose(-2, -1))
        bd = self.rel_shift(torch.matmul((q + self.pos_bias_v).transpose(1, 2), p.transpose(-2, -1)))
        scores = (ac + bd) / math.sqrt(self.d_k)
        scores = scores.masked_fill(~mask[:, None, None, :], float("-inf"))
        att = torch.softmax(scores, dim=-1)
        return self.linear_out(torch.matmul(att, v).transpose(1, 2).reshape(b, t, -1))


class _EspnetCSGU(torch.nn.Module):
    def __init__(self, size, k):
        super().__init__()
        self.norm = torch.nn.LayerNorm(size // 2, eps=1e-6)
        self.conv = torch.nn.Conv1d(size // 2, size // 2, k, 1, (k - 1) // 2, groups=size // 2)
        self.linear = None

    def forward(self, x):
        x_r, x_g = x.chunk(2, dim=-1)
        x_g = self.conv(self.norm(x_g).transpose(1, 2)).transpose(1, 2)
        return x_r * x_g


class _EspnetCGMLP(torch.nn.Module):
    def __init__(self, d, units, k):
        super().__init__()
        self.channel_proj1 = torch.nn.Sequential(torch.nn.Linear(d, units), torch.nn.GELU())
        self.csgu = _EspnetCSGU(units, k)
        self.channel_proj2 = torch.nn.Linear(units // 2, d)

    def forward(self, x):
        return self.channel_proj2(self.csgu(self.channel_proj1(x)))


class _EspnetEBranchformerLayer(torch.nn.Module):
    def __init__(self, d=16, heads=4, ff=24, cgmlp_units=40, cgmlp_kernel=5, merge_kernel=3):
        super().__init__()
        self.feed_forward, self.feed_forward_macaron = _EspnetFF(d, ff), _EspnetFF(d, ff)
        self.attn = _EspnetRelPosMHA(heads, d)
        self.cgmlp = _EspnetCGMLP(d, cgmlp_units, cgmlp_kernel)
        self.norm_ff, self.norm_ff_macaron, self.norm_mha, self.norm_mlp, self.norm_final = (torch.nn.LayerNorm(d, eps=1e-6) for _ in range(5))
        self.depthwise_conv_fusion = torch.nn.Conv1d(2 * d, 2 * d, merge_kernel, 1, (merge_kernel - 1) // 2, groups=2 * d)
        self.merge_proj = torch.nn.Linear(2 * d, d)

    def forward(self, x, pos_emb, mask):
        x = x + 0.5 * self.feed_forward_macaron(self.norm_ff_macaron(x))
        x1 = self.attn(self.norm_mha(x), pos_emb, mask)
        x2 = self.cgmlp(self.norm_mlp(x))
        cat = torch.cat([x1, x2], dim=-1)
        x = x + self.merge_proj(cat + self.depthwise_conv_fusion(cat.transpose(1, 2)).transpose(1, 2))
        x = x + 0.5 * self.feed_forward(self.norm_ff(x))
        return self.norm_final(x)


def _espnet_rel_pos_emb(t, d):
    """ESPnet RelPositionalEncoding: interleaved sin / cos of distances t-1 .. -(t-1)"""
    pos = torch.arange(t - 1, -t, -1.0).unsqueeze(1)
    div = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * -(math.log(10000.0) / d))
    pe = torch.zeros(2 * t - 1, d)
    pe[:, 0::2] = torch.sin(pos * div)
    pe[:, 1::2] = torch.cos(pos * div)
    return pe.unsqueeze(0)


def test_espnet_e_branchformer_layer_import_gives_the_same_output():
    from returnn_b200.frontend.encoder.e_branchformer import EBranchformerLayer
    from returnn_b200.frontend.conversions.espnet_e_branchformer import import_params_espnet_e_branchformer_layer_to_rf

    torch.manual_seed(2)
    src = _EspnetEBranchformerLayer().eval()
    with torch.no_grad():
        for p in src.parameters():
            p.add_(torch.randn_like(p) * 0.1)
    model = Dim(16, name="model")
    layer = EBranchformerLayer(model, ff_dim=24, num_heads=4, cgmlp_ff_dim=20, cgmlp_conv_kernel=5, merge_conv_kernel=3, dropout=0.0, att_dropout=0.0,
                               ff_activation=rf.swish)
    import_params_espnet_e_branchformer_layer_to_rf(src, layer)
    rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)
    t = 9
    time = _time_dim([t])
    x_raw = torch.randn(1, t, 16)
    x = Tensor("x", dims=[batch_dim, time, model], dtype="float32", raw_tensor=x_raw)
    with torch.no_grad():
        got = layer(x, spatial_dim=time).copy_transpose([batch_dim, time, model]).raw_tensor
        ref = src(x_raw, _espnet_rel_pos_emb(t, 16), torch.ones(1, t, dtype=torch.bool))
    assert torch.allclose(got, ref, atol=3e-5), float((got - ref).abs().max())
