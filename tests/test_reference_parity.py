"""
Layers and model-zoo modules against the installed reference package on the CPU: same state-dict keys and shapes, the
reference's randomly initialised parameters loaded into this framework's module, same inputs, outputs equal to 1e-5.
And without the reference: every case batched against one sequence at a time (results must not depend on the padding).

Model code of a case is written once and run with both packages (see ``tests/_parity.py``).
Reference: returnn/frontend/{linear,normalization,conv,attention,rec}.py, encoder/conformer.py, decoder/transformer.py;
the padding-invariance idea is that of tests/rf_utils.py:58-120 (run_model, test_single_batch_entry).
"""

import numpy
import pytest
import torch

import _parity as P

needs_ref = pytest.mark.skipif(not P.reference_available(), reason="reference package not installed under baseline/_ref")

LENS = [11, 7, 4]


class Case:
    """one module: how to build it, how to call it"""

    def __init__(self, name, make, fwd, *, in_feat=6, sparse_vocab=None, atol=1e-5, min_len=1):
        self.name, self.make, self.fwd = name, make, fwd
        self.in_feat, self.sparse_vocab, self.atol, self.min_len = in_feat, sparse_vocab, atol, min_len

    def __repr__(self):
        return self.name


def _make_input(case: Case, lens, seed=3):
    rng = numpy.random.RandomState(seed)
    t = max(lens)
    if case.sparse_vocab:
        x = rng.randint(0, case.sparse_vocab, size=(len(lens), t)).astype("int32")
    else:
        x = rng.standard_normal((len(lens), t, case.in_feat)).astype("float32")
    for b, n in enumerate(lens):
        x[b, n:] = 0
    return x


def run_case(api: P.Api, case: Case, x_np, lens, *, params_from=None):
    """build, optionally load parameters, call; returns (masked output array [B, T', ...], output lengths, env)"""
    api.setup()
    torch.manual_seed(0)
    api.rf.set_random_seed(1)
    env = case.make(api)
    if params_from is not None:
        P.copy_params(params_from[0], params_from[1]["module"], api, env["module"])
    time = api.time_dim(lens)
    if case.sparse_vocab:
        x = api.tensor("x", [api.batch_dim, time], x_np, sparse_dim=env["in_dim"])
    else:
        x = api.tensor("x", [api.batch_dim, time, env["in_dim"]], x_np)
    with torch.no_grad():
        y, out_time = case.fwd(api, env, x, time)
    rest = [d for d in y.dims if d not in (api.batch_dim, out_time)]
    arr = P.to_numpy_bt(api, y, [api.batch_dim, out_time] + rest)
    out_lens = [int(v) for v in out_time.dyn_size_ext.raw_tensor.tolist()] if out_time.dyn_size_ext is not None else [arr.shape[1]] * arr.shape[0]
    return P.masked(arr, out_lens), out_lens, env


# ---- the cases -------------------------------------------------------------------------------------------------------------------

def _linear(api):
    i, o = api.Dim(6, name="in"), api.Dim(5, name="out")
    return {"module": api.rf.Linear(i, o), "in_dim": i}


def _linear_nobias(api):
    i, o = api.Dim(6, name="in"), api.Dim(5, name="out")
    return {"module": api.rf.Linear(i, o, with_bias=False), "in_dim": i}


def _embedding(api):
    v, o = api.Dim(13, name="vocab"), api.Dim(8, name="emb")
    return {"module": api.rf.Embedding(v, o), "in_dim": v}


def _layer_norm(api):
    i = api.Dim(6, name="in")
    return {"module": api.rf.LayerNorm(i), "in_dim": i}


def _batch_norm_eval(api):
    i = api.Dim(6, name="in")
    m = api.rf.BatchNorm(i, use_mask=True)
    return {"module": m, "in_dim": i}


def _conv1d(padding, filter_size=3, strides=None):
    def make(api):
        i, o = api.Dim(6, name="in"), api.Dim(7, name="out")
        return {"module": api.rf.Conv1d(i, o, filter_size, padding=padding, strides=strides), "in_dim": i}

    return make


def _fwd_conv(api, env, x, time):
    y, out_time = env["module"](x, in_spatial_dim=time)
    return y, out_time


def _self_att(api):
    i = api.Dim(8, name="in")
    m = api.rf.SelfAttention(i, proj_dim=api.Dim(8, name="proj"), key_dim_total=api.Dim(8, name="key"), value_dim_total=api.Dim(8, name="val"), num_heads=2)
    return {"module": m, "in_dim": i}


def _rel_pos_self_att(api):
    i = api.Dim(8, name="in")
    m = api.rf.RelPosSelfAttention(i, proj_dim=api.Dim(8, name="proj"), key_dim_total=api.Dim(8, name="key"), value_dim_total=api.Dim(8, name="val"),
                                   num_heads=2, with_bias=False, with_linear_pos=True, with_pos_bias=True, separate_pos_emb_per_head=True)
    return {"module": m, "in_dim": i}


def _fwd_att(api, env, x, time):
    return env["module"](x, axis=time), time


def _lstm(api):
    i, o = api.Dim(6, name="in"), api.Dim(5, name="lstm")
    return {"module": api.rf.LSTM(i, o), "in_dim": i}


def _fwd_lstm(api, env, x, time):
    m = env["module"]
    y, _state = m(x, state=m.default_initial_state(batch_dims=[api.batch_dim]), spatial_dim=time)
    return y, time


def _ff(api):
    i = api.Dim(8, name="in")
    m = api.mod("encoder.conformer").ConformerPositionwiseFeedForward(i, ff_dim=api.Dim(16, name="ff"), dropout=0.1, activation=api.rf.swish)
    return {"module": m, "in_dim": i}


def _conformer_conv_block(api):
    i = api.Dim(8, name="in")
    m = api.mod("encoder.conformer").ConformerConvBlock(i, kernel_size=5, norm=api.rf.BatchNorm(i, use_mask=True))
    return {"module": m, "in_dim": i}


def _fwd_spatial(api, env, x, time):
    return env["module"](x, spatial_dim=time), time


def _conformer_subsample(api):
    i = api.Dim(10, name="in")
    m = api.mod("encoder.conformer").ConformerConvSubsample(
        i, out_dims=[api.Dim(3, name="c1"), api.Dim(4, name="c2"), api.Dim(4, name="c3")], filter_sizes=[(3, 3), (3, 3), (3, 3)],
        pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)])
    return {"module": m, "in_dim": i}


def _fwd_subsample(api, env, x, time):
    y, out_time = env["module"](x, in_spatial_dim=time)
    return y, out_time


def _conformer_layer(api):
    i = api.Dim(8, name="in")
    m = api.mod("encoder.conformer").ConformerEncoderLayer(i, ff_dim=api.Dim(16, name="ff"), num_heads=2, conv_kernel_size=5, dropout=0.1, att_dropout=0.1)
    return {"module": m, "in_dim": i}


def _conformer_encoder(api):
    i = api.Dim(10, name="in")
    C = api.mod("encoder.conformer")
    m = C.ConformerEncoder(
        i, api.Dim(8, name="model"), num_layers=2, num_heads=2, ff_dim=api.Dim(16, name="ff"), conv_kernel_size=5, dropout=0.1, att_dropout=0.1,
        input_layer=C.ConformerConvSubsample(i, out_dims=[api.Dim(3, name="c1"), api.Dim(4, name="c2"), api.Dim(4, name="c3")],
                                             filter_sizes=[(3, 3), (3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)]))
    return {"module": m, "in_dim": i}


def _fwd_encoder(api, env, x, time):
    y, out_time = env["module"](x, in_spatial_dim=time)
    return y, out_time


def _conformer_v2(api):
    i = api.Dim(10, name="in")
    model = api.Dim(8, name="model")
    C, C2 = api.mod("encoder.conformer"), api.mod("encoder.conformer_v2")

    class Both(api.rf.Module):
        def __init__(self):
            super().__init__()
            self.frontend = C2.ConformerFrontend(
                i, model, input_embedding_scale=8 ** 0.5, input_dropout=0.1,
                input_layer=C.ConformerConvSubsample(i, out_dims=[api.Dim(3, name="c1"), api.Dim(4, name="c2")], filter_sizes=[(3, 3), (3, 3)],
                                                     pool_sizes=[(1, 2)], strides=[(1, 1), (2, 1)]))
            self.encoder = C2.ConformerEncoderV2(model, num_layers=2, num_heads=2, ff_dim=api.Dim(16, name="ff"), conv_kernel_size=5,
                                                 encoder_layer_opts={"conv_norm": api.rf.LayerNorm})

        def __call__(self, x, *, in_spatial_dim):
            x, out_time = self.frontend(x, in_spatial_dim=in_spatial_dim)
            return self.encoder(x, spatial_dim=out_time), out_time

    return {"module": Both(), "in_dim": i}


def _e_branchformer_encoder(api):
    i = api.Dim(10, name="in")
    model = api.Dim(8, name="model")
    C, C2, E = api.mod("encoder.conformer"), api.mod("encoder.conformer_v2"), api.mod("encoder.e_branchformer")

    class Both(api.rf.Module):
        def __init__(self):
            super().__init__()
            self.frontend = C2.ConformerFrontend(i, model, input_layer=C.ConformerConvSubsample(
                i, out_dims=[api.Dim(3, name="c1"), api.Dim(4, name="c2")], filter_sizes=[(3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (2, 1)]))
            self.encoder = C2.ConformerEncoderV2(model, num_layers=2, encoder_layer=api.rf.build_dict(
                E.EBranchformerLayer, ff_dim=16, num_heads=2, cgmlp_ff_dim=12, cgmlp_conv_kernel=5, merge_conv_kernel=3))

        def __call__(self, x, *, in_spatial_dim):
            x, out_time = self.frontend(x, in_spatial_dim=in_spatial_dim)
            return self.encoder(x, spatial_dim=out_time), out_time

    return {"module": Both(), "in_dim": i}


def _transformer_encoder(api):
    v = api.Dim(13, name="vocab")
    m = api.mod("encoder.transformer").TransformerEncoder(
        v, api.Dim(8, name="model"), num_layers=2, num_heads=2, dropout=0.1, att_dropout=0.1,
        ff={"class": "returnn.frontend.decoder.transformer.FeedForward", "ff_dim": api.Dim(16, name="ff")})
    return {"module": m, "in_dim": v}


def _fwd_tr_encoder(api, env, x, time):
    return env["module"](x, spatial_dim=time), time


def _transformer_decoder_lm(api):
    v = api.Dim(13, name="vocab")
    m = api.mod("decoder.transformer").TransformerDecoder(None, v, api.Dim(8, name="model"), num_layers=2, num_heads=2, ff_dim=api.Dim(16, name="ff"),
                                                      dropout=0.1, att_dropout=0.1)
    return {"module": m, "in_dim": v}


def _llama_style_decoder(api):
    if api.name == "reference":
        # the reference's default RoPE goes through torch.compile, whose C++ build has no OpenMP spec file on this image; its own
        # eager restatement of the same op (used by the reference whenever it traces statically) takes its place
        import returnn.torch.util.rope as ref_rope

        ref_rope.apply_rope = ref_rope.apply_rope_plain
    v = api.Dim(13, name="vocab")
    D = api.mod("decoder.transformer")
    m = D.TransformerDecoder(
        None, v, api.Dim(8, name="model"), num_layers=2, num_heads=2, pos_enc=None, norm=api.rf.build_dict(api.rf.RMSNorm),
        ff=api.rf.build_dict(D.FeedForwardGated, ff_dim=12), layer_opts=dict(self_att=api.rf.build_dict(api.rf.RotaryPosCausalSelfAttention, with_bias=False)),
        share_embedding=False, dropout=0.1, att_dropout=0.1)
    return {"module": m, "in_dim": v}


def _fwd_decoder_lm(api, env, x, time):
    m = env["module"]
    logits, _state = m(x, spatial_dim=time, state=m.default_initial_state(batch_dims=[api.batch_dim]))
    return logits, time


CASES = [
    Case("linear", _linear, lambda api, env, x, t: (env["module"](x), t)),
    Case("linear_nobias", _linear_nobias, lambda api, env, x, t: (env["module"](x), t)),
    Case("embedding", _embedding, lambda api, env, x, t: (env["module"](x), t), sparse_vocab=13),
    Case("layer_norm", _layer_norm, lambda api, env, x, t: (env["module"](x), t)),
    Case("batch_norm_eval", _batch_norm_eval, lambda api, env, x, t: (env["module"](x), t)),
    Case("conv1d_same", _conv1d("same"), _fwd_conv),
    Case("conv1d_valid", _conv1d("valid"), _fwd_conv, min_len=3),
    Case("conv1d_same_stride2", _conv1d("same", 3, 2), _fwd_conv),
    Case("conv1d_valid_k4_stride3", _conv1d("valid", 4, 3), _fwd_conv, min_len=4),
    Case("self_attention", _self_att, _fwd_att, in_feat=8),
    Case("rel_pos_self_attention", _rel_pos_self_att, _fwd_att, in_feat=8),
    Case("lstm", _lstm, _fwd_lstm),
    Case("conformer_ffn", _ff, lambda api, env, x, t: (env["module"](x), t), in_feat=8),
    Case("conformer_conv_block", _conformer_conv_block, _fwd_spatial, in_feat=8),
    Case("conformer_conv_subsample", _conformer_subsample, _fwd_subsample, in_feat=10, min_len=7),
    Case("conformer_layer", _conformer_layer, _fwd_spatial, in_feat=8, atol=2e-5),
    Case("conformer_encoder", _conformer_encoder, _fwd_encoder, in_feat=10, atol=5e-5, min_len=7),
    Case("conformer_frontend_and_encoder_v2", _conformer_v2, _fwd_encoder, in_feat=10, atol=5e-5, min_len=7),
    Case("e_branchformer_encoder", _e_branchformer_encoder, _fwd_encoder, in_feat=10, atol=5e-5, min_len=7),
    Case("transformer_encoder", _transformer_encoder, _fwd_tr_encoder, sparse_vocab=13, atol=2e-5),
    Case("transformer_decoder_lm", _transformer_decoder_lm, _fwd_decoder_lm, sparse_vocab=13, atol=2e-5),
    Case("llama_style_decoder_rope_rmsnorm_swiglu", _llama_style_decoder, _fwd_decoder_lm, sparse_vocab=13, atol=2e-5),
]


def _lens_for(case: Case):
    return [max(n, case.min_len) + (12 if case.min_len > 4 else 0) for n in LENS]


@needs_ref
@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_module_equals_reference(case):
    """reference-initialised parameters loaded into our module: same keys, same shapes, same outputs"""
    lens = _lens_for(case)
    x = _make_input(case, lens)
    ref_out, ref_lens, ref_env = run_case(P.reference(), case, x, lens)
    our_out, our_lens, _ = run_case(P.ours(), case, x, lens, params_from=(P.reference(), ref_env))
    assert our_lens == ref_lens
    P.assert_close(our_out, ref_out, atol=case.atol, what=case.name)


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_module_padding_invariance(case):
    """each sequence alone gives what it gives inside a padded batch"""
    api = P.ours()
    lens = _lens_for(case)
    x = _make_input(case, lens)
    full, out_lens, env = run_case(api, case, x, lens)
    for b, n in enumerate(lens):
        time = api.time_dim([n])
        xb = x[b: b + 1, :n]
        if case.sparse_vocab:
            xt = api.tensor("x", [api.batch_dim, time], xb, sparse_dim=env["in_dim"])
        else:
            xt = api.tensor("x", [api.batch_dim, time, env["in_dim"]], xb)
        with torch.no_grad():
            y, out_time = case.fwd(api, env, xt, time)
        rest = [d for d in y.dims if d not in (api.batch_dim, out_time)]
        arr = P.to_numpy_bt(api, y, [api.batch_dim, out_time] + rest)
        m = out_lens[b]
        assert arr.shape[1] >= m
        P.assert_close(arr[0, :m], full[b, :m], atol=max(case.atol, 2e-5), what="%s seq %i" % (case.name, b))
