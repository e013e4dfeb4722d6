"""
Static decoder step + graph-replayed beam search (returnn_b200/models/decode_graph.py) against the RF decoder driven by the
ordinary search loop (returnn_b200/models/beam_search.py): same logits per step, same hypotheses, lengths and scores.
"""

import pytest
import torch

import returnn_b200.frontend as rf
from returnn_b200.tensor import Tensor, Dim, batch_dim

gpu = pytest.mark.gpu


def _setup(dev):
    from returnn_b200.frontend.decoder.transformer import TransformerDecoder

    torch.manual_seed(0)
    rf.set_random_seed(7)
    enc_dim, vocab, model = Dim(12, name="enc"), Dim(11, name="vocab"), Dim(16, name="model")
    dec = TransformerDecoder(enc_dim, vocab, model, num_layers=2, num_heads=4, ff_dim=Dim(32, name="ff"), dropout=0.0, att_dropout=0.0)
    for p in dec.parameters():
        p.raw_tensor.data = (p.raw_tensor.data + 0.3 * torch.randn_like(p.raw_tensor.data)).to(dev)
    return dec, enc_dim, vocab, model


def _rf_search(dec, enc_raw, enc_lens, vocab, beam, max_len, bos, eos, dev):
    from returnn_b200.models.beam_search import beam_search_raw
    from returnn_b200.frontend import nested

    B = enc_raw.shape[0]
    beam_batch = Dim(None, name="batch-beam")
    beam_batch.dyn_size_ext = Tensor("bb", dims=[], dtype="int32", raw_tensor=torch.tensor(B * beam, dtype=torch.int32))
    spatial = Dim(None, name="enc-time")
    spatial.dyn_size_ext = Tensor("l", dims=[beam_batch], dtype="int32", raw_tensor=enc_lens.repeat_interleave(beam).to(torch.int32))
    enc_b = Tensor("enc", dims=[beam_batch, spatial, dec.encoder_dim], dtype="float32", raw_tensor=enc_raw.repeat_interleave(beam, dim=0))
    enc_state = dec.transform_encoder(enc_b, axis=spatial)
    state = dec.default_initial_state(batch_dims=[beam_batch])
    logits_log = []

    def step_fn(prev, st):
        lab = Tensor("prev", dims=[beam_batch], dtype="int64", sparse_dim=vocab, raw_tensor=prev)
        logits, st = dec(lab, spatial_dim=rf.single_step_dim, encoder=enc_state, state=st)
        raw = logits.copy_transpose([beam_batch, vocab]).raw_tensor
        logits_log.append(raw.detach().clone())
        return raw, st

    def reorder(st, flat):
        def g(t):
            if isinstance(t, Tensor) and t.raw_tensor is not None and beam_batch in t.dims:
                return rf._utils.wrap(t.raw_tensor.index_select(list(t.dims).index(beam_batch), flat), t.dims, like=t)
            return t

        return nested.tree_map(g, st)

    with torch.no_grad():
        res = beam_search_raw(step_fn, state, reorder, batch=B, beam=beam, vocab=vocab.dimension, bos=bos, eos=eos, max_len=max_len, device=dev)
    return res, logits_log


def _check(dev, use_graph):
    from returnn_b200.models.decode_graph import StaticTransformerDecoderStep, beam_search_static

    dec, enc_dim, vocab, model = _setup(dev)
    rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)
    B, beam, bos, eos = 3, 4, 1, 0
    enc_lens = torch.tensor([9, 5, 7])
    enc_raw = torch.randn(B, 9, 12, device=dev)
    max_len = torch.tensor([7, 4, 6])
    (labels, lens, scores), logits_log = _rf_search(dec, enc_raw, enc_lens, vocab, beam, max_len, bos, eos, dev)
    stepper = StaticTransformerDecoderStep(dec, enc=enc_raw, enc_lens=enc_lens,
                                           num_hyps=B * beam, max_steps=int(max_len.max()))
    # the first step alone: same logits as the RF decoder
    with torch.no_grad():
        first = stepper.step(torch.full((B * beam,), bos, dtype=torch.int64, device=dev))
    torch.testing.assert_close(first.float(), logits_log[0].float(), atol=2e-4, rtol=1e-4)
    with torch.no_grad():
        labels2, lens2, scores2 = beam_search_static(stepper, batch=B, beam=beam, bos=bos, eos=eos, max_len=max_len, use_graph=use_graph, check_every=3)
    torch.testing.assert_close(scores2.cpu(), scores.cpu(), atol=2e-4, rtol=1e-4)
    assert torch.equal(lens2.cpu(), lens.cpu())
    for b in range(B):
        for k in range(beam):
            n = int(lens[b, k])
            assert labels2[b, k, :n].tolist() == labels[b, k, :n].tolist(), (b, k)
    # a second search on the same object starts from a clean state
    with torch.no_grad():
        labels3, lens3, scores3 = beam_search_static(stepper, batch=B, beam=beam, bos=bos, eos=eos, max_len=max_len, use_graph=use_graph)
    torch.testing.assert_close(scores3.cpu(), scores2.cpu(), atol=1e-6, rtol=0)


def test_static_decoder_step_and_search_cpu():
    _check("cpu", use_graph=False)


@gpu
def test_graph_replayed_beam_search_gpu():
    _check("cuda", use_graph=True)


@gpu
@pytest.mark.parametrize("d,group,T", [(64, 1, 40), (64, 4, 161), (128, 3, 70)])
def test_decode_attention_kernel_matches_fp32(d, group, T):
    """the one-query attention kernel (shared cache per group, lengths from a tensor or from the step counter) against an fp32 restatement"""
    import ctypes
    from returnn_b200.ops import _lib

    torch.manual_seed(0)
    nk, H = 5, 3
    N = nk * group
    q = torch.randn(N, H, d, device="cuda").bfloat16()
    k = torch.randn(nk, H, T, d, device="cuda").bfloat16()
    v = torch.randn(nk, H, T, d, device="cuda").bfloat16()
    lens = torch.tensor([T, 1, T // 2, 33, 7], dtype=torch.int32, device="cuda")
    pos = torch.tensor([T // 3], dtype=torch.int64, device="cuda")
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    fn = _lib.bind("rb200_decode_attention", [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, ctypes.c_float, vp, vp])
    for use_lens in (True, False):
        out = torch.empty(N, H, d, dtype=torch.bfloat16, device="cuda")
        _lib.check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr() if use_lens else None, None if use_lens else pos.data_ptr(),
                      N, H, T, d, group, d ** -0.5, out.data_ptr(), _lib.stream_ptr()), "decode_attention")
        valid = lens.repeat_interleave(group) if use_lens else torch.full((N,), int(pos[0]) + 1, device="cuda", dtype=torch.int32)
        kf, vf = k.float().repeat_interleave(group, 0), v.float().repeat_interleave(group, 0)
        scores = torch.einsum("nhd,nhtd->nht", q.float(), kf) * d ** -0.5
        scores = scores.masked_fill(torch.arange(T, device="cuda")[None, None, :] >= valid[:, None, None], float("-inf"))
        ref = torch.einsum("nht,nhtd->nhd", torch.softmax(scores, -1), vf)
        torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)


@gpu
def test_static_step_bf16_native_attention_matches_library_attention():
    """bf16 stepper with 64-dim heads: the own attention kernel and torch's attention give the same logits"""
    import os
    from returnn_b200.frontend.decoder.transformer import TransformerDecoder
    from returnn_b200.models.decode_graph import StaticTransformerDecoderStep

    torch.manual_seed(0)
    rf.set_random_seed(7)
    enc_dim, vocab, model = Dim(24, name="enc"), Dim(50, name="vocab"), Dim(128, name="model")
    dec = TransformerDecoder(enc_dim, vocab, model, num_layers=2, num_heads=2, ff_dim=Dim(64, name="ff"), dropout=0.0, att_dropout=0.0)
    for p in dec.parameters():
        p.raw_tensor.data = p.raw_tensor.data.cuda()
    enc = torch.randn(3, 20, 24, device="cuda")
    enc_lens = torch.tensor([20, 9, 14])
    outs = []
    for disable in (False, True):
        if disable:
            os.environ["RETURNN_B200_DISABLE_NATIVE"] = "1"
        try:
            st = StaticTransformerDecoderStep(dec, enc=enc, enc_lens=enc_lens, num_hyps=12, max_steps=6, dtype=torch.bfloat16)
            prev = torch.arange(12, device="cuda") % 50
            with torch.no_grad():
                logits = [st.step((prev + i) % 50).float() for i in range(4)]
            outs.append(torch.stack(logits))
        finally:
            os.environ.pop("RETURNN_B200_DISABLE_NATIVE", None)
    torch.testing.assert_close(outs[0], outs[1], atol=6e-2, rtol=5e-2)
