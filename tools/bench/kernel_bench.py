"""
Micro-benchmarks of the non-GEMM kernels at the shapes of the flagship Conformer step (packed rows n ~ 6.7k, D = 512):

    python tools/bench/kernel_bench.py [--only NAME] [--iters K] [--rows N]

For every op: device time of forward and of forward+backward (CUDA events around ``iters`` calls, a spin kernel in front so
that the host has queued everything before the first event), the algorithmic bytes it has to move, and the achieved
fraction of the measured HBM copy bandwidth (``MEASURED_PEAKS.json`` next to the repository root if present, else the
fallback 6650 GB/s). One JSON line per op. Used for the kernel summaries under ``profiles/`` (also as the small workload
for ``ncu`` captures: ``--only NAME --iters 2``).
"""

from __future__ import annotations
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import argparse
import json
import os
import torch


def _peak_gbs() -> float:
    fn = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(fn))["hbm_gbs"])
    except Exception:
        return 6650.0


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(int(2e7))
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=6656)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--only", default=None)
    ap.add_argument("--variant", default="", help="op-specific switches, comma separated (decode_step: bf16, static_only)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    n, D, F = args.rows, 512, 2048
    peak = _peak_gbs()
    bf = torch.bfloat16
    from returnn_b200.ops import layer_norm as ln, elementwise as ew, conv_module as cm, ctc as ctc_op, attention_packed as att, softmax_ce as ce, logmel, seq_ops
    from returnn_b200.models.packing import PackInfo

    torch.manual_seed(0)
    lens = torch.randint(60, 334, (64,))
    while int(lens.sum()) > n:
        lens = lens[:-1]
    lens[-1] += n - int(lens.sum())
    pack = PackInfo(lens.to(torch.int32), dev)
    n = pack.n
    results = []

    def report(name, t_fwd, t_fb, bytes_fwd, bytes_fb, extra=None):
        r = {"op": name, "fwd_us": round(t_fwd * 1e6, 1), "fwd_bwd_us": round(t_fb * 1e6, 1) if t_fb else None,
             "fwd_gbs": round(bytes_fwd / t_fwd / 1e9, 1), "fwd_frac_of_measured_hbm": round(bytes_fwd / t_fwd / 1e9 / peak, 3)}
        if t_fb:
            r["fwd_bwd_gbs"] = round(bytes_fb / t_fb / 1e9, 1)
            r["fwd_bwd_frac_of_measured_hbm"] = round(bytes_fb / t_fb / 1e9 / peak, 3)
        if extra:
            r.update(extra)
        results.append(r)
        print(json.dumps(r), flush=True)

    def want(name):
        return args.only is None or args.only == name

    if want("layer_norm"):
        x = torch.randn(n, D, device=dev, dtype=bf, requires_grad=True)
        g = torch.ones(D, device=dev, requires_grad=True)
        b = torch.zeros(D, device=dev, requires_grad=True)
        dy = torch.randn(n, D, device=dev, dtype=bf)
        fwd = lambda: ln.layer_norm(x, g, b, 1e-6)
        def fb():
            y = ln.layer_norm(x, g, b, 1e-6)
            y.backward(dy)
        report("layer_norm", _time(fwd, args.iters), _time(fb, args.iters), 2 * n * D * 2, (2 + 3) * n * D * 2)
    if want("dropout"):
        x = torch.randn(n, F, device=dev, dtype=bf)
        report("dropout", _time(lambda: ew.dropout(x, 0.1), args.iters), None, 2 * n * F * 2, 0)
    if want("conv_module"):
        from returnn_b200.tensor import Dim
        from returnn_b200 import frontend as rf

        bn = rf.BatchNorm(Dim(D, name="c"), use_mask=True)
        for p in bn.parameters():
            p.raw_tensor = p.raw_tensor.to(dev) if p.raw_tensor is not None else None
        for name in ("running_mean", "running_variance"):
            t = getattr(bn, name)
            t.raw_tensor = t.raw_tensor.to(dev)
        x = torch.randn(n, 2 * D, device=dev, dtype=bf, requires_grad=True)
        filt = (torch.randn(D, 1, 32, device=dev) * 0.1).requires_grad_(True)
        bias = torch.zeros(D, device=dev, requires_grad=True)
        dy = torch.randn(n, D, device=dev, dtype=bf)
        fwd = lambda: cm.glu_dwconv_bn_silu(x, filt, bias, bn, pack, training=True)
        def fb():
            cm.glu_dwconv_bn_silu(x, filt, bias, bn, pack, training=True).backward(dy)
        # fwd: read [n,2D], write y and z [n,D] each, re-read y;  bwd: read y, dz, x, ds; write ds, dx
        report("conv_module (GLU+dwconv32+BN+SiLU)", _time(fwd, args.iters), _time(fb, args.iters), (2 + 1 + 1 + 1) * n * D * 2,
               (5 + 1 + 1 + 1 + 1 + 2 + 1 + 2) * n * D * 2)
    if want("rel_pos_attention"):
        H, Dh = 8, 64
        qkv = (torch.randn(n, 3 * H * Dh, device=dev) * 0.3).to(bf).requires_grad_(True)
        L = pack.max_len
        pos = (torch.randn(2 * L - 1, H * Dh, device=dev) * 0.3).to(bf).requires_grad_(True)
        u = torch.zeros(H, Dh, device=dev, requires_grad=True)
        v = torch.zeros(H, Dh, device=dev, requires_grad=True)
        dy = torch.randn(n, H * Dh, device=dev, dtype=bf)
        fwd = lambda: att.rel_pos_attention_packed(qkv, pos, u, v, pack, num_heads=H, head_dim=Dh, scale=Dh ** -0.5, dropout_p=0.1)
        def fb():
            fwd().backward(dy)
        lp = (L + 63) // 64 * 64
        score_bytes = pack.batch * H * lp * lp
        flops = 4.0 * H * Dh * float((lens.double() ** 2).sum()) * 2  # QK^T + bias band + PV, valid part only
        # fwd traffic: scores fp32 write+read, band fp32 (2x wide) write+read, probabilities bf16 write (+dropped copy) + read
        report("rel_pos_attention (packed, 8x64)", _time(fwd, args.iters), _time(fb, args.iters), score_bytes * (8 + 16 + 6) + 5 * n * H * Dh * 2,
               score_bytes * (8 + 16 + 6) * 3, {"fwd_tflops_valid": round(flops / 1e12 / 1.0, 4)})
    if want("ctc"):
        V = 10001
        logits = torch.randn(n, V, device=dev).to(bf).requires_grad_(True)
        tl = torch.clamp((lens.float() / 5).long(), min=1)
        targets = torch.randint(0, V - 1, (pack.batch, int(tl.max())), device=dev, dtype=torch.int32)
        fwd = lambda: ctc_op.ctc_loss_packed(logits, pack, targets, tl, blank_index=V - 1)
        def fb():
            fwd().sum().backward()
        report("ctc (V=10001, packed logits)", _time(fwd, args.iters), _time(fb, args.iters), n * V * 2, n * V * 2 * 3)
    if want("softmax_ce"):
        V = 10240
        logits = torch.randn(n, V, device=dev).to(bf).requires_grad_(True)
        tg = torch.randint(0, V, (n,), device=dev)
        fwd = lambda: ce.softmax_cross_entropy(logits, tg, 0.1)
        def fb():
            fwd().sum().backward()
        report("softmax_ce (V=10240, smoothing)", _time(fwd, args.iters), _time(fb, args.iters), n * V * 2, n * V * 2 * 3)
    if want("log_mel"):
        audio = torch.randn(64, 16000 * 10, device=dev)
        fwd = lambda: logmel.log_mel(audio, sampling_rate=16000, window=400, step=160, n_fft=512, n_mel=80, f_min=0.0, f_max=8000.0)
        frames = (160000 - 400) // 160 + 1
        report("log_mel (64 x 10 s)", _time(fwd, args.iters), None, 64 * 160000 * 4 + 64 * frames * 80 * 4, 0,
               {"gflops_dft": round(64 * frames * 257 * 400 * 4 / 1e9, 1)})
    if want("beam_topk"):
        logits = torch.randn(64, 12, 10001, device=dev).to(bf)
        prev = torch.randn(64, 12, device=dev)
        fwd = lambda: seq_ops.beam_topk(logits, prev, eos=0, k=12)
        report("beam_topk (64 x 12 x 10001)", _time(fwd, args.iters), None, 64 * 12 * 10001 * 2 * 2, 0)
    import ctypes
    from returnn_b200.ops import _lib

    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    if want("layer_norm_bwd_acc"):
        # the form the training step uses: bf16 rows, residual gradient added, dgamma / dbeta accumulated in the kernel
        x = torch.randn(n, D, device=dev, dtype=bf)
        dy = torch.randn(n, D, device=dev, dtype=bf)
        dres = torch.randn(n, D, device=dev, dtype=bf)
        dx = torch.empty_like(x)
        gam = torch.ones(D, device=dev)
        mean = x.float().mean(1).contiguous()
        rstd = (x.float().var(1, unbiased=False) + 1e-6).rsqrt().contiguous()
        dg, db = torch.zeros(D, device=dev), torch.zeros(D, device=dev)
        part = torch.empty(2 * 592 * D, device=dev)
        fn = _lib.bind("rb200_layer_norm_bwd_ex", [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, vp, i32, vp])
        call = lambda: _lib.check(fn(x.data_ptr(), dy.data_ptr(), gam.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), part.data_ptr(),
                                     dg.data_ptr(), db.data_ptr(), n, D, 416, 1, 0, 0, dres.data_ptr(), 1, _lib.stream_ptr()), "ln_bwd")
        report("layer_norm_bwd_acc (bf16, + residual gradient)", _time(call, args.iters), None, 4 * n * D * 2, 0)
    if want("colsum"):
        for width in (D, F):
            x = torch.randn(n, width, device=dev, dtype=bf)
            out = torch.zeros(width, device=dev)
            fn = _lib.bind("rb200_colsum_bf16", [vp, vp, i32, i32, vp])
            call = lambda: _lib.check(fn(x.data_ptr(), out.data_ptr(), n, width, _lib.stream_ptr()), "colsum")
            report("colsum (bias gradient, %i columns)" % width, _time(call, args.iters), None, n * width * 2, 0)
    if want("att_softmax_bf16"):
        H = 8
        L = pack.max_len
        lp = (L + 63) // 64 * 64
        rp = 2 * lp
        B = pack.batch
        s_ac = (torch.randn(B * H * lp, lp, device=dev) * 2).to(bf)
        band = (torch.randn(H * B * lp, rp, device=dev) * 2).to(bf)
        w = torch.empty(B * H * lp, lp, device=dev, dtype=bf)
        wd = torch.empty_like(w)
        seed = torch.tensor([1234, 0], device=dev, dtype=torch.int64)
        off = torch.zeros(1, device=dev, dtype=torch.int64)
        lens_dev = pack.lens
        fwd_fn = _lib.bind("rb200_att_softmax_fwd_ex", [vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp, vp, vp])
        fwd = lambda: _lib.check(fwd_fn(s_ac.data_ptr(), band.data_ptr(), 1, w.data_ptr(), wd.data_ptr(), lens_dev.data_ptr(), B, H, lp, rp, lp - 1, 0.1,
                                        seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "att_softmax_fwd")
        dwd = torch.randn(B * H * lp, lp, device=dev).to(bf)
        ds = torch.empty_like(w)
        dband = torch.zeros(H * B * lp, rp, device=dev, dtype=bf)
        bwd_fn = _lib.bind("rb200_att_softmax_bwd_ex", [vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp, vp, vp])
        bwd = lambda: _lib.check(bwd_fn(w.data_ptr(), dwd.data_ptr(), 1, ds.data_ptr(), dband.data_ptr(), lens_dev.data_ptr(), B, H, lp, rp, lp - 1, 0.1,
                                        seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "att_softmax_bwd")
        valid = float((lens.double() ** 2).sum()) * H
        t_f = _time(fwd, args.iters)
        fwd()
        t_b = _time(bwd, args.iters)
        report("att_softmax fwd (bf16 scores, dropout)", t_f, None, valid * 2 * 4, 0)
        report("att_softmax bwd (bf16 scores, dropout)", t_b, None, valid * 2 * 4, 0)
    if want("adamw"):
        # the optimizer step of the flagship model: one kernel over the flat arena of 82.4 M fp32 parameters; per element it reads
        # parameter, gradient and both moments and writes parameter, both moments and the bf16 copy of the parameter (30 bytes)
        from returnn_b200.ops import optim_native

        n_par = 82387968
        p_ = torch.randn(n_par, device=dev) * 0.05
        g_ = torch.randn(n_par, device=dev) * 0.01
        m_ = torch.zeros(n_par, device=dev)
        v_ = torch.zeros(n_par, device=dev)
        p16 = torch.empty(n_par, device=dev, dtype=bf)
        flags = torch.ones(n_par // 4, device=dev, dtype=torch.uint8)
        norm = torch.full((1,), 3.0, device=dev)
        step = lambda: optim_native.adamw_arena(p_, g_, m_, v_, flags, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, bc1=0.1, bc2=0.001, decoupled=True,
                                                clip=5.0, norm=norm, p_bf16=p16)
        report("adamw (82.4 M parameters, clip factor on the fly, bf16 copy)", _time(step, args.iters), None, n_par * 30, 0)
    if want("sdpa"):
        # scaled dot-product attention of the Transformer models: 64 sequences x 256 positions, 8 heads x 64, bf16, causal and with key lengths
        from returnn_b200.ops import sdpa as sdpa_op

        Bs, Ts, Hs, Ds = 64, 256, 8, 64
        q_ = (torch.randn(Bs, Ts, Hs * Ds, device=dev) * 0.5).to(bf).requires_grad_(True)
        k_ = (torch.randn(Bs, Ts, Hs * Ds, device=dev) * 0.5).to(bf).requires_grad_(True)
        v_ = (torch.randn(Bs, Ts, Hs * Ds, device=dev) * 0.5).to(bf).requires_grad_(True)
        kl = torch.randint(Ts // 2, Ts + 1, (Bs,), dtype=torch.int32)
        dy_ = torch.randn(Bs, Ts, Hs * Ds, device=dev).to(bf)
        for name_, kw in (("sdpa (key lengths)", dict(k_lens=kl)), ("sdpa (causal)", dict(causal=True))):
            fwd = lambda kw=kw: sdpa_op.sdpa(q_, k_, v_, num_heads=Hs, **kw)
            def fb(fwd=fwd):
                fwd().backward(dy_)
            flops = 4.0 * Bs * Hs * Ts * Ts * Ds
            report(name_ + " 64 x 256, 8 x 64", _time(fwd, args.iters), _time(fb, args.iters), 4 * Bs * Ts * Hs * Ds * 2, 9 * Bs * Ts * Hs * Ds * 2,
                   {"fwd_gflop": round(flops / 1e9, 1)})
    if want("rnnt"):
        # RNN-T loss over the [T, U+1] lattice of every sequence: 32 sequences, T = 200 frames, U = 50 labels
        Br, Tr, Ur = 32, 200, 50
        lp_b = torch.log_softmax(torch.randn(Br, Tr, Ur + 1, 2, device=dev), -1)
        lpb = lp_b[..., 0].contiguous().requires_grad_(True)
        lpl = lp_b[..., 1].contiguous().requires_grad_(True)
        t_l = torch.full((Br,), Tr, dtype=torch.int32)
        u_l = torch.full((Br,), Ur, dtype=torch.int32)
        fwd = lambda: seq_ops.rnnt_loss(lpb, lpl, t_l, u_l)
        def fb():
            fwd().sum().backward()
        report("rnnt_loss (32 x 200 x 51 lattice)", _time(fwd, args.iters), _time(fb, args.iters), 2 * Br * Tr * (Ur + 1) * 4, 6 * Br * Tr * (Ur + 1) * 4)
    if want("decode_step"):
        # one label of beam search with a 6 x 512 Transformer decoder (8 heads, ff 2048, vocabulary 10k), 32 sequences x beam 12:
        # the RF step interface driven from Python against one CUDA-graph replay per label over static caches
        import time
        from returnn_b200.tensor import Tensor, Dim
        from returnn_b200 import frontend as rf
        from returnn_b200.frontend.decoder.transformer import TransformerDecoder
        from returnn_b200.frontend import nested
        from returnn_b200.models.beam_search import beam_search_raw
        from returnn_b200.models.decode_graph import StaticTransformerDecoderStep, beam_search_static

        Bq, beam, t_enc, n_lab = 32, 12, 160, 40
        enc_dim, vocab, model = Dim(512, name="enc"), Dim(10000, name="vocab"), Dim(512, name="model")
        dec = TransformerDecoder(enc_dim, vocab, model, num_layers=6, num_heads=8, ff_dim=Dim(2048, name="ff"), dropout=0.0, att_dropout=0.0)
        for p_ in dec.parameters():
            p_.raw_tensor.data = p_.raw_tensor.data.to(dev)
        rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)
        enc_raw = torch.randn(Bq * beam, t_enc, 512, device=dev)
        enc_lens = torch.full((Bq * beam,), t_enc, dtype=torch.int32)
        max_len = torch.full((Bq,), n_lab, dtype=torch.int64)
        bb = Dim(None, name="bb")
        bb.dyn_size_ext = Tensor("bb", dims=[], dtype="int32", raw_tensor=torch.tensor(Bq * beam, dtype=torch.int32))
        sp = Dim(None, name="enc-time")
        sp.dyn_size_ext = Tensor("l", dims=[bb], dtype="int32", raw_tensor=enc_lens)

        def rf_search():
            enc_state = dec.transform_encoder(Tensor("enc", dims=[bb, sp, enc_dim], dtype="float32", raw_tensor=enc_raw), axis=sp)

            def step_fn(prev, st):
                lab = Tensor("prev", dims=[bb], dtype="int64", sparse_dim=vocab, raw_tensor=prev)
                logits, st = dec(lab, spatial_dim=rf.single_step_dim, encoder=enc_state, state=st)
                return logits.copy_transpose([bb, vocab]).raw_tensor, st

            def reorder(st, flat):
                return nested.tree_map(lambda t: rf._utils.wrap(t.raw_tensor.index_select(list(t.dims).index(bb), flat), t.dims, like=t)
                                       if isinstance(t, Tensor) and t.raw_tensor is not None and bb in t.dims else t, st)

            # eos = a label the random model practically never prefers, so that all n_lab labels are decoded
            return beam_search_raw(step_fn, dec.default_initial_state(batch_dims=[bb]), reorder, batch=Bq, beam=beam, vocab=10000, bos=1, eos=0,
                                   max_len=max_len, device=dev)

        variants = set(v for v in args.variant.split(",") if v)
        with torch.no_grad(), torch.autocast("cuda", dtype=bf, enabled="bf16" in variants):
            stepper = StaticTransformerDecoderStep(dec, enc=enc_raw[::beam].contiguous(), enc_lens=enc_lens[::beam].contiguous(), num_hyps=Bq * beam, max_steps=n_lab,
                                                   dtype=bf if "bf16" in variants else None)
            res = {}
            forms = (("rf_loop", rf_search), ("static_graph", lambda: beam_search_static(stepper, batch=Bq, beam=beam, bos=1, eos=0, max_len=max_len)))
            if "static_only" in variants:
                forms = forms[1:]
                res["rf_loop"] = (0.0, 1)
            for name, fn_ in forms:
                fn_()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                out_ = fn_()
                torch.cuda.synchronize()
                res[name] = ((time.perf_counter() - t0) * 1e3, int(out_[1].max()))
        r = {"op": "beam search label step (6x512 decoder, 32 x 12 hypotheses, vocab 10k)",
             "rf_loop_ms_per_label": round(res["rf_loop"][0] / max(res["rf_loop"][1], 1), 3), "rf_loop_labels": res["rf_loop"][1],
             "static_graph_ms_per_label": round(res["static_graph"][0] / max(res["static_graph"][1], 1), 3), "static_graph_labels": res["static_graph"][1],
             "dtype": "bf16" if "bf16" in variants else "fp32",
             "note": "wall clock of the second search (the static form replays the graph captured by the first) / labels decoded"}
        print(json.dumps(r), flush=True)
    if want("lstm"):
        from returnn_b200.ops import lstm_native

        for (T, Bl) in ((400, 48), (1600, 12)):
            Hl, I = 1024, 2048
            x = (torch.randn(T, Bl, I, device=dev) * 0.5).to(bf).requires_grad_(True)
            w_ff = (torch.randn(4 * Hl, I, device=dev) * 0.02).requires_grad_(True)
            w_rec = (torch.randn(4 * Hl, Hl, device=dev) * 0.02).requires_grad_(True)
            bias = torch.zeros(4 * Hl, device=dev, requires_grad=True)
            h0, c0 = torch.zeros(Bl, Hl, device=dev), torch.zeros(Bl, Hl, device=dev)
            ll = torch.full((Bl,), T, dtype=torch.int32)
            fwd = lambda: lstm_native.lstm(x, ll, w_ff, w_rec, bias, h0, c0, reverse=False)[0]
            def fb():
                fwd().float().sum().backward()
            t_f, t_fb = _time(fwd, max(2, args.iters // 10)), _time(fb, max(2, args.iters // 10))
            report("lstm layer T=%i B=%i H=1024 (input GEMM + persistent recurrence)" % (T, Bl), t_f, t_fb, T * Bl * (I + 5 * Hl) * 2, T * Bl * (I + 5 * Hl) * 2 * 3,
                   {"fwd_us_per_step": round(t_f * 1e6 / T, 2), "bwd_us_per_step": round((t_fb - t_f) * 1e6 / T, 2)})
            # both directions of a bidirectional layer: one launch for the two time loops against two launches in a row
            w2 = [(torch.randn(4 * Hl, I, device=dev) * 0.02).requires_grad_(True), (torch.randn(4 * Hl, Hl, device=dev) * 0.02).requires_grad_(True),
                  torch.zeros(4 * Hl, device=dev, requires_grad=True)]
            if lstm_native.blstm_supported(x, w_rec, w2[1]):
                from returnn_b200.ops import lstm as lstm_ops

                def pair():
                    (yf, _, _), (yb, _, _) = lstm_ops.blstm(x, ll, (w_ff, w_rec, bias), tuple(w2), h0, c0, h0, c0)
                    return yf, yb

                def seq():
                    return (lstm_native.lstm(x, ll, w_ff, w_rec, bias, h0, c0, reverse=False)[0], lstm_native.lstm(x, ll, *w2, h0, c0, reverse=True)[0])

                def fb_of(f):
                    def run():
                        a, b = f()
                        (a.float().sum() + b.float().sum()).backward()
                    return run

                n_it = max(2, args.iters // 10)
                tp_f, tp_fb = _time(pair, n_it), _time(fb_of(pair), n_it)
                ts_f, ts_fb = _time(seq, n_it), _time(fb_of(seq), n_it)
                report("blstm layer T=%i B=%i H=1024, both directions in one kernel" % (T, Bl), tp_f, tp_fb, 2 * T * Bl * (I + 5 * Hl) * 2,
                       2 * T * Bl * (I + 5 * Hl) * 2 * 3, {"two_launches_fwd_ms": round(ts_f * 1e3, 3), "two_launches_fwd_bwd_ms": round(ts_fb * 1e3, 3),
                                                            "speedup_fwd": round(ts_f / tp_f, 2), "speedup_fwd_bwd": round(ts_fb / tp_fb, 2)})
    from returnn_b200.ops import gemm as G

    G.check_status()


if __name__ == "__main__":
    main()
