"""
Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op.
"""

import math
import pytest
import torch

gpu = pytest.mark.gpu


def _need_lib():
    from returnn_b200.ops import _lib

    assert torch.cuda.is_available()
    assert _lib.get_lib(required=True) is not None


@gpu
@pytest.mark.parametrize("rows,n", [(1, 8), (37, 512), (1000, 512), (129, 2048), (33, 1000), (5, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rms", [False, True])
def test_layer_norm_fwd_bwd(rows, n, dtype, rms):
    _need_lib()
    from returnn_b200.ops import layer_norm as ln

    torch.manual_seed(0)
    x = (torch.randn(rows, n, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
    g = (torch.rand(n, device="cuda") + 0.5).requires_grad_(True)
    b = torch.randn(n, device="cuda").requires_grad_(True)
    dy = torch.randn(rows, n, device="cuda").to(dtype)
    fn = ln.rms_norm if rms else ln.layer_norm
    ref_fn = ln.rms_norm_reference if rms else ln.layer_norm_reference
    n0 = _launches()
    y = fn(x, g, b, 1e-6)
    if n <= 2048:
        assert _launches() > n0, "native kernel did not run"
    y.backward(dy)
    dx, dg, db = x.grad.clone(), g.grad.clone(), b.grad.clone()
    x32 = x.detach().float().requires_grad_(True)
    g32 = g.detach().clone().requires_grad_(True)
    b32 = b.detach().clone().requires_grad_(True)
    y_ref = ref_fn(x32, g32, b32, 1e-6)
    y_ref.backward(dy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(y.float(), y_ref, atol=tol, rtol=tol)
    torch.testing.assert_close(dx.float(), x32.grad, atol=tol * 4, rtol=tol * 2)
    scale = max(1.0, math.sqrt(rows))
    torch.testing.assert_close(dg, g32.grad, atol=tol * scale, rtol=tol * 2)
    torch.testing.assert_close(db, b32.grad, atol=tol * scale, rtol=tol * 2)


def _launches():
    from returnn_b200.ops import _lib

    return _lib.launch_count()


@gpu
@pytest.mark.parametrize("n", [1, 127, 4096, 1_000_003])
def test_sum_squares(n):
    _need_lib()
    from returnn_b200.ops import optim_native

    torch.manual_seed(1)
    x = torch.randn(n, device="cuda")
    scratch = torch.zeros(1100, device="cuda")
    got = optim_native.sum_squares(x, scratch)
    ref = x.double().square().sum()
    assert abs(got.item() - ref.item()) <= 1e-4 * max(1.0, ref.item())


@gpu
@pytest.mark.parametrize("decoupled", [True, False])
def test_fused_arena_adamw_matches_torch(decoupled):
    _need_lib()
    from returnn_b200.torch.optim.fused_adamw import FusedArenaAdamW

    torch.manual_seed(2)

    def make():
        m = torch.nn.Sequential(torch.nn.Linear(33, 65), torch.nn.LayerNorm(65), torch.nn.Linear(65, 7)).cuda()
        return m

    m1 = make()
    m2 = make()
    m2.load_state_dict(m1.state_dict())
    wd_names = {"0.weight", "2.weight"}
    opt1 = FusedArenaAdamW(m1, lr=1e-2, betas=(0.9, 0.98), eps=1e-8, weight_decay=0.1, decoupled=decoupled, weight_decay_param_names=wd_names)
    cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    opt2 = cls([{"params": [m2[0].weight, m2[2].weight], "weight_decay": 0.1},
                {"params": [m2[0].bias, m2[1].weight, m2[1].bias, m2[2].bias], "weight_decay": 0.0}], lr=1e-2, betas=(0.9, 0.98), eps=1e-8)
    for step in range(5):
        x = torch.randn(16, 33, device="cuda")
        for m, opt in ((m1, opt1), (m2, opt2)):
            opt.zero_grad()
            m(x).square().mean().backward()
        if step == 2:
            norm = opt1.grad_norm()
            ref_norm = torch.nn.utils.clip_grad_norm_(m2.parameters(), 0.05)
            torch.testing.assert_close(norm, ref_norm, atol=1e-5, rtol=1e-4)
            opt1.set_clip(0.05, norm)
        opt1.step()
        opt2.step()
    for (n1, p1), (n2, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        torch.testing.assert_close(p1, p2, atol=2e-6, rtol=1e-5, msg=lambda s: "%s: %s" % (n1, s))
    sd = opt1.state_dict()
    assert set(sd["state"][0].keys()) == {"step", "exp_avg", "exp_avg_sq"}


@gpu
def test_dropout_mask_replay_and_rate():
    _need_lib()
    from returnn_b200.ops import elementwise as ew

    x = torch.ones(1 << 20, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ew.dropout(x, 0.25)
    keep = (y.float() != 0).float().mean().item()
    assert abs(keep - 0.75) < 5e-3
    assert torch.all((y == 0) | ((y.float() - 1.0 / 0.75).abs() < 1e-2))
    y.backward(torch.ones_like(y))
    # backward re-creates exactly the forward mask
    assert torch.equal(x.grad != 0, y != 0)
    y2 = ew.dropout(x, 0.25)
    assert not torch.equal(y2 != 0, y != 0), "a second call must draw a new mask"


@gpu
@pytest.mark.parametrize("rows,v", [(7, 10001), (64, 32000), (3, 13)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("smoothing", [0.0, 0.1])
def test_softmax_ce(rows, v, dtype, smoothing):
    _need_lib()
    from returnn_b200.ops import softmax_ce as ce

    torch.manual_seed(3)
    logits = (torch.randn(rows, v, device="cuda") * 3).to(dtype).requires_grad_(True)
    tgt = torch.randint(0, v, (rows,), device="cuda", dtype=torch.int32)
    w = torch.rand(rows, device="cuda")
    loss = ce.softmax_cross_entropy(logits, tgt, smoothing)
    (loss * w).sum().backward()
    l32 = logits.detach().float().requires_grad_(True)
    ref = ce.softmax_cross_entropy_reference(l32, tgt, smoothing)
    (ref * w).sum().backward()
    torch.testing.assert_close(loss, ref, atol=2e-3, rtol=1e-4)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(logits.grad.float(), l32.grad, atol=tol, rtol=tol)


@gpu
@pytest.mark.parametrize("rows,v", [(9, 10001), (32, 32000)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_softmax_ce_smoothed_gradient_and_argmax(rows, v, dtype):
    """loss = NLL, gradient smoothed uniformly over V; arg max per row from the same pass"""
    _need_lib()
    from returnn_b200.ops import softmax_ce as ce

    torch.manual_seed(5)
    logits = (torch.randn(rows, v, device="cuda") * 3).to(dtype).requires_grad_(True)
    tgt = torch.randint(0, v, (rows,), device="cuda", dtype=torch.int32)
    w = torch.rand(rows, device="cuda")
    loss, best = ce.softmax_cross_entropy(logits, tgt, 0.1, grad_only_smoothing=True, with_argmax=True)
    (loss * w).sum().backward()
    l32 = logits.detach().float().requires_grad_(True)
    ref = ce.softmax_cross_entropy_reference(l32, tgt, 0.1, grad_only_smoothing=True)
    (ref * w).sum().backward()
    torch.testing.assert_close(loss, ref, atol=2e-3, rtol=1e-4)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(logits.grad.float(), l32.grad, atol=tol, rtol=tol)
    assert torch.equal(best.long(), logits.detach().float().argmax(dim=-1))


@gpu
def test_log_mel_kernel_matches_stft_path():
    """fused log-mel kernel against the RF path (torch.fft) on the same audio"""
    from returnn_b200.tensor import Tensor, Dim, batch_dim
    import returnn_b200.frontend as rf
    from returnn_b200.ops import logmel

    torch.manual_seed(0)
    audio = torch.randn(3, 16000, device="cuda") * 0.3 + torch.sin(torch.arange(16000, device="cuda") * 0.05)[None]
    t = Dim(None, name="samples")
    t.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([16000, 16000, 16000], dtype=torch.int32))
    x = Tensor("a", dims=[batch_dim, t], dtype="float32", raw_tensor=audio)
    out_dim = Dim(80, name="mel")
    got, _ = rf.audio.log_mel_filterbank_from_raw(x, in_spatial_dim=t, out_dim=out_dim)
    import os

    os.environ["RETURNN_B200_DISABLE_NATIVE"] = "1"
    try:
        x_cpu = Tensor("a", dims=[batch_dim, t], dtype="float32", raw_tensor=audio.cpu())
        ref, _ = rf.audio.log_mel_filterbank_from_raw(x_cpu, in_spatial_dim=t, out_dim=out_dim)
    finally:
        del os.environ["RETURNN_B200_DISABLE_NATIVE"]
    assert tuple(got.raw_tensor.shape) == tuple(ref.raw_tensor.shape) == (3, 98, 80)
    torch.testing.assert_close(got.raw_tensor.cpu(), ref.raw_tensor, atol=2e-3, rtol=2e-3)


def _log_mel_fp64(audio, lens, *, window, step, n_fft, n_mel, sampling_rate=16000):
    """float64 restatement: frames -> Hann window -> rfft -> power -> mel -> log10"""
    from returnn_b200.frontend.audio.mel import _fbank_matrix

    win = torch.hann_window(window, periodic=True, dtype=torch.float64)
    fb = torch.from_numpy(_fbank_matrix(sampling_rate, n_fft, 0.0, sampling_rate / 2.0, n_mel)).double()
    rows, T = audio.shape
    n_frames = (T - window) // step + 1
    frames = audio.double().unfold(1, window, step)[:, :n_frames] * win
    power = torch.fft.rfft(frames, n=n_fft).abs() ** 2
    out = torch.log10(torch.clamp(power @ fb, min=1e-10))
    for r, n in enumerate(lens):
        out[r, max((int(n) - window) // step + 1, 0):] = 0
    return out.float()


def test_log_mel_dft_table_layout_cpu():
    """the packed DFT table (X_0 and X_{N/2} share the first column pair) and the mel filter ranges, checked in float64 on the CPU"""
    from returnn_b200.ops import logmel
    from returnn_b200.frontend.audio.mel import _fbank_matrix

    window, n_fft, n_mel = 400, 512, 80
    win = torch.hann_window(window, periodic=True, dtype=torch.float32)
    fb = torch.from_numpy(_fbank_matrix(16000, n_fft, 0.0, 8000.0, n_mel))
    t_hi, t_lo, start, length = logmel._dft_tables(torch.device("cpu"), window, n_fft, win, fb)
    table = t_hi.double() + t_lo.double()
    x = torch.randn(5, window, dtype=torch.float64)
    spec = x @ table
    ref = torch.fft.rfft(x * win.double(), n=n_fft)
    assert torch.allclose(spec[:, 0], ref[:, 0].real, atol=2e-3) and torch.allclose(spec[:, 1], ref[:, n_fft // 2].real, atol=2e-3)
    assert torch.allclose(spec[:, 2::2], ref[:, 1:n_fft // 2].real, atol=2e-3) and torch.allclose(spec[:, 3::2], ref[:, 1:n_fft // 2].imag, atol=2e-3)
    for m in range(n_mel):
        nz = torch.nonzero(fb[:, m]).flatten()
        assert int(start[m]) == int(nz[0]) and int(start[m] + length[m]) == int(nz[-1]) + 1


@gpu
def test_log_mel_gemm_form_matches_float64():
    """tensor-core DFT (fp16 hi/lo split, three products) against float64, on a signal with about 80 dB between its strongest and weakest band"""
    import os
    from returnn_b200.ops import logmel

    torch.manual_seed(0)
    rows, T = 24, 16000 * 2 + 37
    tt = torch.arange(T, device="cuda")
    audio = torch.sin(tt * 0.05)[None] * 0.8 + torch.randn(rows, T, device="cuda") * 3e-5
    lens = torch.tensor([T] * (rows - 2) + [T // 2, 300], dtype=torch.int32)
    ref = _log_mel_fp64(audio.cpu(), lens, window=400, step=160, n_fft=512, n_mel=80)
    kw = dict(sampling_rate=16000, window=400, step=160, n_fft=512, n_mel=80, f_min=0.0, f_max=8000.0, lens=lens)
    old = os.environ.get("RETURNN_B200_LOGMEL")
    try:
        os.environ["RETURNN_B200_LOGMEL"] = "gemm"
        got = logmel.log_mel(audio, **kw).cpu()
        os.environ["RETURNN_B200_LOGMEL"] = "direct"
        direct = logmel.log_mel(audio, **kw).cpu()
    finally:
        if old is None:
            del os.environ["RETURNN_B200_LOGMEL"]
        else:
            os.environ["RETURNN_B200_LOGMEL"] = old
    assert got.shape == ref.shape == direct.shape
    assert float(ref.max() - ref[:rows - 2].min()) > 7.0  # the test signal really spans > 70 dB in the mel domain
    torch.testing.assert_close(direct, ref, atol=5e-3, rtol=0)
    torch.testing.assert_close(got, ref, atol=5e-3, rtol=0)
    assert float(got[-1].abs().max()) == 0.0 and float(got[-2, (T // 2 - 400) // 160 + 1:].abs().max()) == 0.0


@gpu
@pytest.mark.parametrize("rows,n", [(1, 512), (37, 256), (4100, 512), (9475, 384), (2368 * 5 + 3, 512)])
@pytest.mark.parametrize("with_res", [False, True])
def test_layer_norm_bwd_accumulating_kernel_matches_fp32(rows, n, with_res):
    """the backward the native encoder uses (bf16 rows, residual gradient added, dgamma / dbeta added onto fp32 buffers) against torch in fp32"""
    import ctypes
    from returnn_b200.ops import _lib

    torch.manual_seed(rows + n)
    dev = "cuda"
    bf = torch.bfloat16
    x = (torch.randn(rows, n, device=dev) * 1.5 + 0.3).to(bf)
    dy = torch.randn(rows, n, device=dev).to(bf)
    dres = torch.randn(rows, n, device=dev).to(bf) if with_res else None
    gam = torch.randn(n, device=dev) * 0.5 + 1.0
    xf = x.float().requires_grad_(True)
    gf = gam.clone().requires_grad_(True)
    bias = torch.zeros(n, device=dev, requires_grad=True)
    mean = xf.detach().mean(1).contiguous()
    rstd = (xf.detach().var(1, unbiased=False) + 1e-6).rsqrt().contiguous()
    y = torch.nn.functional.layer_norm(xf, (n,), gf, bias, eps=1e-6)
    y.backward(dy.float())
    dg0, db0 = torch.randn(n, device=dev), torch.randn(n, device=dev)
    dg, db = dg0.clone(), db0.clone()
    dx = torch.empty_like(x)
    part = torch.empty(2 * 592 * n, device=dev)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn = _lib.bind("rb200_layer_norm_bwd_ex", [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, vp, i32, vp])
    _lib.check(fn(x.data_ptr(), dy.data_ptr(), gam.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), part.data_ptr(), dg.data_ptr(), db.data_ptr(),
                  rows, n, 416, 1, 0, 0, dres.data_ptr() if with_res else None, 1, _lib.stream_ptr()), "ln_bwd")
    torch.cuda.synchronize()
    want_dx = xf.grad + (dres.float() if with_res else 0.0)
    torch.testing.assert_close(dx.float(), want_dx, atol=0.03, rtol=0.02)
    scale = max(1.0, rows ** 0.5)
    torch.testing.assert_close(dg - dg0, gf.grad, atol=2e-3 * scale, rtol=1e-3)
    torch.testing.assert_close(db - db0, bias.grad, atol=2e-3 * scale, rtol=1e-3)


@gpu
@pytest.mark.parametrize("bt,m,k,n", [(6, 128, 64, 72), (3, 64, 192, 256), (1, 37, 40, 24), (5, 70, 64, 64)])
def test_batched_matmul_on_own_gemm(bt, m, k, n):
    """ops.bmm (what rf.matmul runs for batched bf16 products): result and both gradients against fp32 torch; shapes outside its rules fall back"""
    from returnn_b200.ops import bmm as B, gemm

    torch.manual_seed(bt * 1000 + m)
    a = (torch.randn(bt, m, k, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(bt, k, n, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    own = B.supported(a, b)
    assert own == (bt == 1 or (k % 64 == 0 and m % 64 == 0))
    launches0 = __import__("returnn_b200.ops._lib", fromlist=["x"]).launch_count()
    c = B.bmm(a, b)
    w = torch.randn(bt, m, n, device="cuda")
    (c.float() * w).sum().backward()
    gemm.check_status()
    launches = __import__("returnn_b200.ops._lib", fromlist=["x"]).launch_count() - launches0
    assert launches == (3 if own else 0)
    ga, gb = a.grad.float().clone(), b.grad.float().clone()
    af, bf_ = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    ref = torch.matmul(af, bf_)
    (ref * w).sum().backward()
    torch.testing.assert_close(c.float(), ref, atol=0.06, rtol=0.02)
    for g, r in ((ga, af.grad), (gb, bf_.grad)):
        assert float((g - r).abs().max()) / (float(r.abs().max()) + 1e-6) < 0.02


@gpu
def test_rf_matmul_batched_uses_own_gemm():
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Tensor, Dim
    from returnn_b200.ops import _lib

    b_, h, t, d = Dim(2, name="b"), Dim(4, name="h"), Dim(128, name="t"), Dim(64, name="d")
    t2 = Dim(192, name="t2")
    q = Tensor("q", dims=[b_, h, t, d], dtype="bfloat16", raw_tensor=torch.randn(2, 4, 128, 64, device="cuda").to(torch.bfloat16))
    k = Tensor("k", dims=[b_, h, t2, d], dtype="bfloat16", raw_tensor=torch.randn(2, 4, 192, 64, device="cuda").to(torch.bfloat16))
    n0 = _lib.launch_count()
    e = rf.matmul(q, k, reduce=d)
    assert _lib.launch_count() == n0 + 1 and e.dims == (b_, h, t, t2)
    ref = torch.matmul(q.raw_tensor.float(), k.raw_tensor.float().transpose(-1, -2))
    torch.testing.assert_close(e.raw_tensor.float(), ref, atol=0.1, rtol=0.02)


@gpu
def test_linear_with_output_width_off_the_pitch_rule_runs_on_the_own_gemm():
    """10001 classes: zero-padded to 10008 on the own GEMM, cut back; values and gradients as torch in fp32"""
    from returnn_b200.ops import linear as L, _lib, gemm

    torch.manual_seed(8)
    x = (torch.randn(300, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(256, 1001, device="cuda") * 0.1).requires_grad_(True)
    b = (torch.randn(1001, device="cuda") * 0.1).requires_grad_(True)
    n0 = _lib.launch_count()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = L.linear(x, w, b)
    assert y.shape == (300, 1001) and _lib.launch_count() > n0
    g = torch.randn(300, 1001, device="cuda")
    (y.float() * g).sum().backward()
    gemm.check_status()
    got = [t.grad.float().clone() for t in (x, w, b)]
    xf, wf, bf_ = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    ref = xf @ wf + bf_
    (ref * g).sum().backward()
    torch.testing.assert_close(y.float(), ref, atol=0.05, rtol=0.02)
    for a, r in zip(got, (xf.grad, wf.grad, bf_.grad)):
        assert float((a - r).abs().max()) / (float(r.abs().max()) + 1e-6) < 0.02
