"""
RF layers and model zoo on CPU: shapes, gradients, and the padding-invariance property of the reference's test suite
(outputs of a sequence do not depend on how much padding the batch carries; reference: tests/rf_utils.py run_model).
"""

import pytest
import torch
from returnn_b200.tensor import Tensor, Dim, batch_dim
import returnn_b200.frontend as rf
from returnn_b200.utils.basic import BehaviorVersion


def _seq(lens, feat, seed=0, extra_pad=0):
    torch.manual_seed(seed)
    t = Dim(None, name="time")
    t.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor(lens, dtype=torch.int32))
    batch_dim.dyn_size_ext = Tensor("batch", dims=[], dtype="int32", raw_tensor=torch.tensor(len(lens), dtype=torch.int32))
    T = max(lens)
    raw = torch.randn(len(lens), T, feat.dimension)
    if extra_pad:
        raw = torch.cat([raw, torch.randn(len(lens), extra_pad, feat.dimension) * 50.0], dim=1)
    for b, n in enumerate(lens):
        raw[b, n:] = torch.randn_like(raw[b, n:]) * 50.0  # garbage in the padding
    return Tensor("x", dims=[batch_dim, t, feat], dtype="float32", raw_tensor=raw), t


def _valid(y: Tensor, t: Dim, lens):
    y = y.copy_transpose([batch_dim, t] + [d for d in y.dims if d not in (batch_dim, t)])
    return [y.raw_tensor[b, :n] for b, n in enumerate(lens)]


def test_linear_layernorm_shapes_and_grad():
    f, o = Dim(8, name="in"), Dim(5, name="out")
    lin, ln = rf.Linear(f, o), rf.LayerNorm(o)
    x, t = _seq([4, 2], f)
    y = ln(lin(x))
    assert y.dims == (batch_dim, t, o)
    loss = rf.reduce_sum(y * y, axis=list(y.dims))
    loss.raw_tensor.backward()
    assert lin.weight.raw_tensor.grad is not None and torch.isfinite(lin.weight.raw_tensor.grad).all()


def test_conformer_padding_invariance():
    BehaviorVersion._reset(24)  # from 23 on, convolution and pooling mask their input (rf.use_mask_default)
    from returnn_b200.frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample

    torch.manual_seed(1)
    f = Dim(16, name="feat")
    model_dim = Dim(32, name="model")
    enc = ConformerEncoder(
        f, model_dim, num_layers=2, num_heads=2, ff_dim=Dim(64, name="ff"), conv_kernel_size=5, dropout=0.0, att_dropout=0.0,
        input_layer=ConformerConvSubsample(f, out_dims=[Dim(4, name="c1"), Dim(4, name="c2")], filter_sizes=[(3, 3), (3, 3)],
                                           pool_sizes=[(1, 2)], strides=[(1, 1), (2, 1)]))
    lens = [24, 13]
    x1, t1 = _seq(lens, f, seed=5)
    # the same two sequences in a batch with a third, longer one: more padding for both
    lens2 = [24, 13, 36]  # same parity as 24: the "same" padding of the strided conv depends on the padded length
    x2, t2 = _seq(lens2, f, seed=6)
    for b, n in enumerate(lens):
        x2.raw_tensor[b, :n] = x1.raw_tensor[b, :n]
    enc.eval() if hasattr(enc, "eval") else None
    with torch.no_grad():
        rf.init_forward_step_run_ctx()
        y1, s1 = enc(x1, in_spatial_dim=t1)
        y2, s2 = enc(x2, in_spatial_dim=t2)
    out_lens = s1.dyn_size_ext.raw_tensor.tolist()
    assert out_lens == s2.dyn_size_ext.raw_tensor.tolist()[:2] == [12, 7]
    for a, b in zip(_valid(y1, s1, out_lens), _valid(y2, s2, out_lens)):
        torch.testing.assert_close(a, b, atol=1e-4, rtol=1e-4)


def test_transformer_decoder_step_equals_full():
    from returnn_b200.frontend.decoder.transformer import TransformerDecoder

    torch.manual_seed(2)
    vocab = Dim(11, name="vocab")
    enc_dim = Dim(16, name="enc")
    dec = TransformerDecoder(encoder_dim=enc_dim, vocab_dim=vocab, model_dim=Dim(16, name="dec"), num_layers=2, num_heads=2, dropout=0.0,
                             att_dropout=0.0)
    enc_x, enc_t = _seq([5, 3], enc_dim, seed=3)
    tgt_t = Dim(None, name="tgt")
    tgt_t.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([4, 4], dtype=torch.int32))
    labels = Tensor("y", dims=[batch_dim, tgt_t], dtype="int32", sparse_dim=vocab, raw_tensor=torch.randint(0, 11, (2, 4), dtype=torch.int32))
    with torch.no_grad():
        rf.init_forward_step_run_ctx()
        enc_state = dec.transform_encoder(enc_x, axis=enc_t)
        full, _ = dec(labels, spatial_dim=tgt_t, encoder=enc_state, state=dec.default_initial_state(batch_dims=[batch_dim]))
        state = dec.default_initial_state(batch_dims=[batch_dim])
        steps = []
        for i in range(4):
            lab_i = Tensor("yi", dims=[batch_dim], dtype="int32", sparse_dim=vocab, raw_tensor=labels.raw_tensor[:, i])
            out_i, state = dec(lab_i, spatial_dim=rf.single_step_dim, encoder=enc_state, state=state)
            steps.append(out_i.copy_transpose([batch_dim, out_i.dims[-1]]).raw_tensor)
    full_raw = full.copy_transpose([batch_dim, tgt_t, full.dims[-1]]).raw_tensor
    torch.testing.assert_close(torch.stack(steps, dim=1), full_raw, atol=1e-4, rtol=1e-4)


def test_lstm_matches_reference_math():
    from returnn_b200.ops import lstm as lstm_ops

    torch.manual_seed(3)
    f, h = Dim(6, name="in"), Dim(5, name="hid")
    lstm = rf.LSTM(f, h)
    x, t = _seq([7, 4], f, seed=4)
    rf.init_forward_step_run_ctx()
    y, state = lstm(x, spatial_dim=t, state=lstm.default_initial_state(batch_dims=[batch_dim]))
    assert y.dims_set == {batch_dim, t, h}
    assert state.h.dims_set == {batch_dim, h}
    # final state of the short sequence is the state at its own last frame, not at the padded end
    y_bt = y.copy_transpose([batch_dim, t, h]).raw_tensor
    torch.testing.assert_close(state.h.copy_transpose([batch_dim, h]).raw_tensor[1], y_bt[1, 3], atol=1e-5, rtol=1e-5)


def test_ctc_loss_against_torch():
    torch.manual_seed(4)
    v = Dim(6, name="wb")
    x, t = _seq([9, 6], v, seed=7)
    s = Dim(None, name="s")
    s.dyn_size_ext = Tensor("sl", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([3, 2], dtype=torch.int32))
    tg = Tensor("t", dims=[batch_dim, s], dtype="int32", sparse_dim=Dim(5, name="lab"), raw_tensor=torch.tensor([[1, 2, 1], [3, 3, 0]], dtype=torch.int32))
    loss = rf.ctc_loss(logits=x, targets=tg, input_spatial_dim=t, targets_spatial_dim=s, blank_index=5)
    lp = torch.log_softmax(x.raw_tensor, -1).transpose(0, 1)
    ref = torch.nn.functional.ctc_loss(lp, tg.raw_tensor.long(), torch.tensor([9, 6]), torch.tensor([3, 2]), blank=5, reduction="none")
    torch.testing.assert_close(loss.raw_tensor, ref, atol=1e-4, rtol=1e-4)


def test_softmax_cross_entropy_smoothed_grad_equals_composition():
    """the one-call criterion equals log_softmax -> label_smoothed_log_prob_gradient -> cross_entropy (value and gradient)"""
    torch.manual_seed(0)
    time_dim = Dim(None, name="time")
    time_dim.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([5, 3], dtype=torch.int32))
    vocab = Dim(11, name="vocab")
    raw = torch.randn(2, 5, 11, requires_grad=True)
    raw2 = raw.detach().clone().requires_grad_(True)
    tgt = Tensor("t", dims=[batch_dim, time_dim], dtype="int64", sparse_dim=vocab, raw_tensor=torch.randint(0, 11, (2, 5)))
    logits = Tensor("x", dims=[batch_dim, time_dim, vocab], dtype="float32", raw_tensor=raw)
    loss, best = rf.softmax_cross_entropy_smoothed_grad(logits=logits, target=tgt, axis=vocab, smoothing=0.1, with_argmax=True)
    logits2 = Tensor("x", dims=[batch_dim, time_dim, vocab], dtype="float32", raw_tensor=raw2)
    lp = rf.log_softmax(logits2, axis=vocab)
    lp = rf.label_smoothed_log_prob_gradient(lp, 0.1, axis=vocab)
    ref = rf.cross_entropy(target=tgt, estimated=lp, estimated_type="log-probs", axis=vocab)
    torch.testing.assert_close(loss.raw_tensor, ref.copy_compatible_to_dims_raw(loss.dims))
    w = torch.rand(2, 5)
    (loss.raw_tensor * w).sum().backward()
    (ref.copy_compatible_to_dims_raw(loss.dims) * w).sum().backward()
    torch.testing.assert_close(raw.grad, raw2.grad, atol=1e-6, rtol=1e-5)
    assert torch.equal(best.raw_tensor, rf.reduce_argmax(logits2, axis=vocab).copy_compatible_to_dims_raw(best.dims))
    assert best.sparse_dim == vocab


def test_random_journal_and_npz_checkpoints(tmp_path):
    """draws recorded in one run come back in another; parameters round-trip through .npz and from an engine-style .pt file"""
    import numpy
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Dim

    a, b = Dim(3, name="a"), Dim(5, name="b")
    journal = rf.RandomJournal()
    with journal.recording():
        x1 = rf.random_normal([a, b])
        u1 = rf.random_uniform([b], minval=-2.0, maxval=2.0)
    assert len(journal) == 2
    rf.set_random_seed(12345)  # another generator state: without the journal the draws would differ
    with journal.replaying():
        x2 = rf.random_normal([a, b])
        u2 = rf.random_uniform([b], minval=-2.0, maxval=2.0)
        assert journal.reached_end()
        with pytest.raises(IndexError):
            rf.random_normal([a])
    assert torch.equal(x1.raw_tensor, x2.raw_tensor) and torch.equal(u1.raw_tensor, u2.raw_tensor)
    with journal.replaying():
        with pytest.raises(ValueError):
            rf.random_normal([b, a])  # other shape than recorded
    # dropout draws through rf.random: the same mask in two runs
    rf.init_train_step_run_ctx(train_flag=True, step=0, epoch=1)
    ones = rf.ones([a, b])
    j2 = rf.RandomJournal()
    with j2.recording():
        d1 = rf.dropout(ones, 0.5, axis=b)
    if len(j2):
        with j2.replaying():
            d2 = rf.dropout(ones, 0.5, axis=b)
        assert torch.equal(d1.raw_tensor, d2.raw_tensor)
    # checkpoints
    lin = rf.Linear(a, b)
    params = rf.checkpoint.get_model_params(lin)
    fn = str(tmp_path / "ck.npz")
    rf.checkpoint.save_params(params, fn, step=7, epoch=2)
    back = rf.checkpoint.load_params(fn)
    assert sorted(back) == ["bias", "weight"] and int(rf.checkpoint.load_params(fn, with_meta=True)["_step"]) == 7
    lin2 = rf.Linear(a, b)
    assert rf.checkpoint.set_model_params(lin2, back) == ["weight", "bias"] or set(rf.checkpoint.set_model_params(lin2, back)) == {"weight", "bias"}
    assert torch.equal(lin2.weight.raw_tensor, lin.weight.raw_tensor)
    with pytest.raises(ValueError):
        rf.checkpoint.check_params_complete(lin2, {"weight": back["weight"]})
    assert rf.checkpoint.check_params_complete(lin2, {"weight": back["weight"]}, allow_missing=True) == ["weight"]
    with pytest.raises(ValueError):
        rf.checkpoint.check_params_complete(lin2, dict(back, extra=numpy.zeros(1)))
    with pytest.raises(ValueError):
        rf.checkpoint.check_params_complete(lin2, dict(back, weight=numpy.zeros((5, 3), dtype="float32")))
    from returnn_b200.torch.frontend.bridge import rf_module_to_pt_module

    pt_fn = str(tmp_path / "model.pt")
    torch.save({"model": rf_module_to_pt_module(lin).state_dict(), "epoch": 3, "step": 11}, pt_fn)
    from_pt = rf.checkpoint.load_torch_checkpoint(pt_fn)
    assert numpy.array_equal(from_pt["weight"], params["weight"]) and numpy.array_equal(from_pt["bias"], params["bias"])
