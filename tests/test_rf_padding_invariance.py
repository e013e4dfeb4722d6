"""Every RF op and module that looks along a dynamic axis: the result on valid frames must not depend on what the padding holds or how much of it there is."""

import pytest
import torch

import returnn_b200.frontend as rf
from returnn_b200.tensor import Tensor, Dim, batch_dim
from returnn_b200.utils.basic import BehaviorVersion
from rf_utils import make_batch, check_padding_invariance

F = Dim(6, name="feat")
LENS = [9, 4, 7, 1]


def _lin(out=5, seed=0):
    torch.manual_seed(seed)
    return rf.Linear(F, Dim(out, name="out"))


# name -> function (x, time) -> (y, out_time or None). Modules are built once per case (same parameters for all calls).
def _cases():
    c = {}
    c["reduce_sum"] = lambda: lambda x, t: (rf.reduce_sum(x, axis=t), None)
    c["reduce_mean"] = lambda: lambda x, t: (rf.reduce_mean(x, axis=t), None)
    c["reduce_max"] = lambda: lambda x, t: (rf.reduce_max(x, axis=t), None)
    c["reduce_min"] = lambda: lambda x, t: (rf.reduce_min(x, axis=t), None)
    c["reduce_logsumexp"] = lambda: lambda x, t: (rf.reduce_logsumexp(x * 0.01, axis=t), None)
    c["reduce_argmax"] = lambda: lambda x, t: (rf.reduce_argmax(x, axis=t), None)
    c["reduce_argmin"] = lambda: lambda x, t: (rf.reduce_argmin(x, axis=t), None)
    c["reduce_sum_two_axes"] = lambda: lambda x, t: (rf.reduce_sum(x, axis=[t, F]), None)
    c["softmax_over_time"] = lambda: lambda x, t: (rf.softmax(x, axis=t), t)
    c["log_softmax_over_time"] = lambda: lambda x, t: (rf.log_softmax(x, axis=t), t)
    c["softmax_over_feature"] = lambda: lambda x, t: (rf.softmax(x, axis=F), t)
    c["cumsum"] = lambda: lambda x, t: (rf.cumsum(x, spatial_dim=t), t)
    c["reverse_sequence"] = lambda: lambda x, t: (rf.reverse_sequence(x, axis=t), t)
    c["top_k_over_time"] = lambda: lambda x, t: (rf.top_k(x, axis=t, k=1)[0], None)
    c["matmul_reduce_time"] = lambda: lambda x, t: (rf.matmul(x, x, reduce=t), None)
    c["linear"] = lambda: (lambda m: lambda x, t: (m(x), t))(_lin())
    c["layer_norm"] = lambda: (lambda m: lambda x, t: (m(x), t))(rf.LayerNorm(F))
    c["rms_norm"] = lambda: (lambda m: lambda x, t: (m(x), t))(rf.RMSNorm(F))
    c["batch_norm_eval"] = lambda: (lambda m: lambda x, t: (m(x), t))(rf.BatchNorm(F, use_mask=True))
    c["group_norm"] = lambda: (lambda m: lambda x, t: (m(x), t))(rf.GroupNorm(F, num_groups=2)) if hasattr(rf, "GroupNorm") else None
    c["conv1d_same"] = lambda: (lambda m: lambda x, t: m(x, in_spatial_dim=t))(rf.Conv1d(F, Dim(5, name="c"), 3, padding="same"))
    c["conv1d_valid"] = lambda: (lambda m: lambda x, t: m(x, in_spatial_dim=t))(rf.Conv1d(F, Dim(5, name="c"), 1, padding="valid"))
    c["conv1d_same_stride2"] = lambda: (lambda m: lambda x, t: m(x, in_spatial_dim=t))(rf.Conv1d(F, Dim(5, name="c"), 3, padding="same", strides=2))
    c["conv1d_depthwise"] = lambda: (lambda m: lambda x, t: m(x, in_spatial_dim=t))(rf.Conv1d(F, F, 5, padding="same", groups=F.dimension))
    c["max_pool1d"] = lambda: lambda x, t: rf.max_pool1d(x, pool_size=2, padding="same", in_spatial_dim=t)
    c["avg_pool1d"] = lambda: lambda x, t: rf.pool1d(x, mode="avg", pool_size=3, padding="same", in_spatial_dim=t)
    c["pool1d_strided"] = lambda: lambda x, t: rf.pool1d(x, mode="max", pool_size=2, strides=2, padding="same", in_spatial_dim=t)
    c["lstm"] = lambda: (lambda m: lambda x, t: (m(x, state=m.default_initial_state(batch_dims=[batch_dim]), spatial_dim=t)[0], t))(
        rf.LSTM(F, Dim(4, name="lstm")))
    c["lstm_final_state"] = lambda: (lambda m: lambda x, t: (m(x, state=m.default_initial_state(batch_dims=[batch_dim]), spatial_dim=t)[1].c, None))(
        rf.LSTM(F, Dim(4, name="lstm")))
    c["self_attention"] = lambda: (lambda m: lambda x, t: (m(x, axis=t), t))(
        rf.SelfAttention(F, proj_dim=F, key_dim_total=Dim(8, name="k"), value_dim_total=Dim(8, name="v"), num_heads=2, att_dropout=0.0))
    c["causal_self_attention"] = lambda: (lambda m: lambda x, t: (m(x, axis=t, state=m.default_initial_state(batch_dims=[batch_dim]))[0], t))(
        rf.CausalSelfAttention(F, proj_dim=F, key_dim_total=Dim(8, name="k"), value_dim_total=Dim(8, name="v"), num_heads=2, att_dropout=0.0))
    c["rel_pos_self_attention"] = lambda: (lambda m: lambda x, t: (m(x, axis=t), t))(
        rf.RelPosSelfAttention(F, proj_dim=F, key_dim_total=Dim(8, name="k"), value_dim_total=Dim(8, name="v"), num_heads=2, att_dropout=0.0))
    c["sinusoidal_positional_encoding_added"] = lambda: lambda x, t: (x + rf.sinusoidal_positional_encoding(spatial_dim=t, feat_dim=F), t)
    c["window"] = lambda: lambda x, t: (rf.window(x, spatial_dim=t, window_dim=Dim(3, name="w"))[0], t)
    c["shift_right"] = lambda: lambda x, t: (rf.shift_right(x, axis=t, pad_value=0.0), t)
    c["pad_then_reduce"] = lambda: lambda x, t: (lambda p: (rf.reduce_sum(p[0], axis=p[1][0]), None))(rf.pad(x, axes=[t], padding=[(1, 2)], value=0.5, handle_dynamic_dims=True))
    c["stack_frames_slice"] = lambda: lambda x, t: rf.slice(x, axis=t, start=1)
    c["concat_time"] = lambda: lambda x, t: (lambda r: (rf.reduce_sum(r[0], axis=r[1]), None))(rf.concat((x, t), (x, t), handle_dynamic_dims=True))
    c["gather_last_frame"] = lambda: lambda x, t: (rf.gather(x, indices=rf.copy_to_device(t.get_dyn_size_ext_for_device(None)) - 1, axis=t), None)
    c["sequence_mask_where"] = lambda: lambda x, t: (rf.reduce_sum(rf.where(rf.sequence_mask([batch_dim, t]), x, 0.0), axis=t, use_mask=False), None)
    c["dropout_eval"] = lambda: lambda x, t: (rf.dropout(x, 0.5, axis=F), t)
    c["relu_square_gelu_chain"] = lambda: lambda x, t: (rf.gelu(rf.relu(x) - rf.sigmoid(x)), t)
    c["cross_entropy_mean"] = lambda: lambda x, t: (
        rf.reduce_mean(rf.cross_entropy(estimated=x * 0.01, estimated_type="logits", target=rf.reduce_argmax(x, axis=F), axis=F), axis=t), None)
    c["ctc_loss"] = lambda: lambda x, t: (_ctc(x, t), None)
    c["conformer_conv_block"] = lambda: (lambda m: lambda x, t: (m(x, spatial_dim=t), t))(_conv_block())
    c["conformer_layer"] = lambda: (lambda m: lambda x, t: (m(x, spatial_dim=t), t))(_conformer_layer())
    c["transformer_encoder_layer"] = lambda: (lambda m: lambda x, t: (m(x, spatial_dim=t), t))(_transformer_layer())
    c["feed_forward"] = lambda: (lambda m: lambda x, t: (m(x), t))(_ff())
    return c


def _ctc(x, t):
    vocab = Dim(F.dimension, name="labels")
    lens = t.dyn_size_ext.raw_tensor
    tgt_len = torch.clamp(lens // 3, min=1)
    s = Dim(None, name="tgt")
    s.dyn_size_ext = Tensor("tl", dims=[batch_dim], dtype="int32", raw_tensor=tgt_len.to(torch.int32))
    g = torch.Generator().manual_seed(int(lens.sum()))
    # targets derived from the sequence itself (so that the single-sequence call sees the same ones): argmax of the first frames, no blank
    first = x.raw_tensor[:, : int(tgt_len.max()), 1:].argmax(-1) + 1
    targets = Tensor("y", dims=[batch_dim, s], dtype="int64", sparse_dim=vocab, raw_tensor=first)
    logits = Tensor("l", dims=[batch_dim, t, vocab], dtype="float32", raw_tensor=x.raw_tensor * 0.01, feature_dim=vocab)
    return rf.ctc_loss(logits=logits, logits_normalized=False, targets=targets, input_spatial_dim=t, targets_spatial_dim=s, blank_index=0)


def _conv_block():
    from returnn_b200.frontend.encoder.conformer import ConformerConvBlock

    torch.manual_seed(3)
    return ConformerConvBlock(F, kernel_size=5, norm=rf.BatchNorm(F, use_mask=True))


def _conformer_layer():
    from returnn_b200.frontend.encoder.conformer import ConformerEncoderLayer

    torch.manual_seed(4)
    return ConformerEncoderLayer(F, ff_dim=Dim(12, name="ff"), num_heads=2, conv_kernel_size=3, dropout=0.0, att_dropout=0.0,
                                 conv_norm=rf.build_dict(rf.BatchNorm, use_mask=True))


def _transformer_layer():
    from returnn_b200.frontend.encoder.transformer import TransformerEncoderLayer

    torch.manual_seed(5)
    return TransformerEncoderLayer(F, ff_dim=Dim(12, name="ff"), num_heads=2, dropout=0.0, att_dropout=0.0)


def _ff():
    from returnn_b200.frontend.encoder.conformer import ConformerPositionwiseFeedForward

    torch.manual_seed(6)
    return ConformerPositionwiseFeedForward(F, ff_dim=Dim(12, name="ff"), dropout=0.0, activation=rf.swish)


_CASES = _cases()


@pytest.mark.parametrize("name", sorted(_CASES))
def test_padding_invariance(name):
    BehaviorVersion._reset(24)
    make = _CASES[name]
    fn = make()
    if fn is None:
        pytest.skip("not in this build")
    x, t = make_batch(LENS, F, seed=11)
    check_padding_invariance(fn, x, t, atol=2e-5, rtol=1e-4, train_flag=name.endswith("_train"))


def test_harness_catches_a_leak():
    """an unmasked torch reduction over the padded axis must be reported"""
    x, t = make_batch(LENS, F, seed=12)

    def leaky(x, t):
        raw = x.copy_transpose([batch_dim, t, F]).raw_tensor.sum(1)
        return Tensor("y", dims=[batch_dim, F], dtype="float32", raw_tensor=raw), None

    with pytest.raises(AssertionError):
        check_padding_invariance(leaky, x, t)


@pytest.mark.parametrize("lens", [[5], [1, 1], [3, 8, 8, 2, 6]])
def test_embedding_and_sparse_inputs(lens):
    vocab = Dim(11, name="vocab")
    torch.manual_seed(7)
    emb = rf.Embedding(vocab, F)
    x, t = make_batch(lens, None, seed=3, dtype="int64", sparse_dim=vocab)
    check_padding_invariance(lambda x, t: (rf.reduce_sum(emb(x), axis=t), None), x, t)
    check_padding_invariance(lambda x, t: (rf.one_hot(x), t), x, t)


def test_batch_norm_training_statistics_ignore_padding():
    """batch statistics in training are over the valid frames only: they come out as mean 0 / variance 1 although the padding holds values around 1500"""
    BehaviorVersion._reset(24)
    bn = rf.BatchNorm(F, use_mask=True, track_running_stats=False, eps=1e-9)
    x, t = make_batch(LENS, F, seed=21)
    rf.init_train_step_run_ctx(train_flag=True, step=0, epoch=1)
    with torch.no_grad():
        y = bn(x).copy_transpose([batch_dim, t, F]).raw_tensor
    valid = torch.cat([y[b, :n] for b, n in enumerate(LENS)])
    torch.testing.assert_close(valid.mean(0), torch.zeros(F.dimension), atol=1e-5, rtol=0)
    torch.testing.assert_close(valid.var(0, unbiased=False), torch.ones(F.dimension), atol=1e-4, rtol=0)
    # the unmasked variant is what leaks: its statistics are dominated by the padding
    bn_unmasked = rf.BatchNorm(F, use_mask=False, track_running_stats=False)
    with torch.no_grad():
        y_u = bn_unmasked(x).copy_transpose([batch_dim, t, F]).raw_tensor
    valid_u = torch.cat([y_u[b, :n] for b, n in enumerate(LENS)])
    assert float(valid_u.mean().abs()) > 0.3
