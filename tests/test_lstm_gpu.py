"""LSTM recurrence executor against the step-by-step fp32 torch reference: outputs, final states and all gradients, both directions."""

import pytest
import torch

gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("T,B,I,H", [(9, 5, 16, 32), (40, 12, 64, 128), (30, 40, 64, 256), (12, 50, 32, 128)])
def test_lstm_native_matches_reference(reverse, T, B, I, H):
    from returnn_b200.ops import lstm as L, lstm_native, gemm

    torch.manual_seed(0)
    dev = "cuda"
    x = (torch.randn(T, B, I, device=dev) * 0.5).requires_grad_(True)
    w_ff = (torch.randn(4 * H, I, device=dev) * 0.2).requires_grad_(True)
    w_rec = (torch.randn(4 * H, H, device=dev) * 0.2).requires_grad_(True)
    bias = (torch.randn(4 * H, device=dev) * 0.1).requires_grad_(True)
    h0 = (torch.randn(B, H, device=dev) * 0.3).requires_grad_(True)
    c0 = (torch.randn(B, H, device=dev) * 0.3).requires_grad_(True)
    lens = torch.randint(1, T + 1, (B,))
    lens[0] = T
    wy = torch.randn(T, B, H, device=dev)
    wh, wc = torch.randn(B, H, device=dev), torch.randn(B, H, device=dev)
    args = (x, w_ff, w_rec, bias, h0, c0)
    assert lstm_native.available(x) and lstm_native.supports(x, w_rec)
    y, h, c = lstm_native.lstm(x, lens, w_ff, w_rec, bias, h0, c0, reverse=reverse)
    ((y.float() * wy).sum() + (h.float() * wh).sum() + (c.float() * wc).sum()).backward()
    gemm.check_status()
    got = [t.grad.clone() for t in args]
    for t in args:
        t.grad = None
    yr, hr, cr = L.lstm_reference(x, lens, w_ff, w_rec, bias, h0, c0, reverse=reverse)
    ((yr * wy).sum() + (hr * wh).sum() + (cr * wc).sum()).backward()
    torch.testing.assert_close(y.float(), yr, atol=0.03, rtol=0.03)
    torch.testing.assert_close(h.float(), hr, atol=0.03, rtol=0.03)
    torch.testing.assert_close(c.float(), cr, atol=0.05, rtol=0.03)
    for name, g, t in zip(("x", "w_ff", "w_rec", "bias", "h0", "c0"), got, args):
        scale = float(t.grad.abs().max()) + 1e-6
        err = float((g.float() - t.grad).abs().max()) / scale
        assert err < 0.06, "gradient of %s: rel. max err %.4f" % (name, err)


@gpu
@pytest.mark.parametrize("T,B,I,H", [(40, 12, 64, 128), (30, 40, 64, 256), (21, 16, 128, 1024)])
def test_blstm_one_kernel_for_both_directions_matches_reference(T, B, I, H):
    """the two-direction persistent kernel: outputs, final states and all gradients of both directions against the fp32 step loop"""
    from returnn_b200.ops import lstm as L, lstm_native, gemm

    torch.manual_seed(1)
    dev = "cuda"
    x = (torch.randn(T, B, I, device=dev) * 0.5).requires_grad_(True)

    def params():
        return [(torch.randn(4 * H, I, device=dev) * 0.2).requires_grad_(True), (torch.randn(4 * H, H, device=dev) * (0.2 if H < 1024 else 0.05)).requires_grad_(True),
                (torch.randn(4 * H, device=dev) * 0.1).requires_grad_(True)]

    fw, bw = params(), params()
    states = [(torch.randn(B, H, device=dev) * 0.3).requires_grad_(True) for _ in range(4)]
    lens = torch.randint(1, T + 1, (B,))
    lens[0] = T
    wts = [torch.randn(T, B, H, device=dev) for _ in range(2)] + [torch.randn(B, H, device=dev) for _ in range(4)]
    leaves = [x] + fw + bw + states
    assert lstm_native.blstm_supported(x, fw[1], bw[1])
    (yf, hf, cf), (yb, hb, cb) = L.blstm(x, lens, tuple(fw), tuple(bw), *states)
    outs = (yf, yb, hf, cf, hb, cb)
    sum((o.float() * w).sum() for o, w in zip(outs, wts)).backward()
    gemm.check_status()
    got = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    yfr, hfr, cfr = L.lstm_reference(x, lens, *fw, states[0], states[1], reverse=False)
    ybr, hbr, cbr = L.lstm_reference(x, lens, *bw, states[2], states[3], reverse=True)
    refs = (yfr, ybr, hfr, cfr, hbr, cbr)
    sum((o * w).sum() for o, w in zip(refs, wts)).backward()
    for o, r in zip(outs, refs):
        torch.testing.assert_close(o.float(), r, atol=0.05, rtol=0.03)
    names = ["x", "fw.w_ff", "fw.w_rec", "fw.bias", "bw.w_ff", "bw.w_rec", "bw.bias", "h0_fw", "c0_fw", "h0_bw", "c0_bw"]
    for name, g, t in zip(names, got, leaves):
        scale = float(t.grad.abs().max()) + 1e-6
        err = float((g.float() - t.grad).abs().max()) / scale
        assert err < 0.06, "gradient of %s: rel. max err %.4f" % (name, err)


@gpu
@pytest.mark.parametrize("T,B,I,H", [(25, 96, 64, 128), (18, 130, 32, 256)])
def test_blstm_large_batch_runs_in_chunks_of_the_persistent_kernel(T, B, I, H):
    """more sequences than one launch of the persistent kernels takes: groups of sequences, each over its own longest length"""
    from returnn_b200.ops import lstm as L, gemm

    torch.manual_seed(2)
    dev = "cuda"
    x = (torch.randn(T, B, I, device=dev) * 0.5).requires_grad_(True)

    def params():
        return [(torch.randn(4 * H, I, device=dev) * 0.2).requires_grad_(True), (torch.randn(4 * H, H, device=dev) * 0.2).requires_grad_(True),
                (torch.randn(4 * H, device=dev) * 0.1).requires_grad_(True)]

    fw, bw = params(), params()
    states = [(torch.randn(B, H, device=dev) * 0.3).requires_grad_(True) for _ in range(4)]
    lens = torch.sort(torch.randint(1, T + 1, (B,)), descending=True).values
    lens[0] = T
    chunks = L._batch_chunks(x, lens, fw[1], bw[1])
    assert chunks is not None and len(chunks) == -(-B // L.PERSIST_MAX_ROWS) and chunks[-1][2] < T
    wts = [torch.randn(T, B, H, device=dev) for _ in range(2)] + [torch.randn(B, H, device=dev) for _ in range(4)]
    leaves = [x] + fw + bw + states
    (yf, hf, cf), (yb, hb, cb) = L.blstm(x, lens, tuple(fw), tuple(bw), *states)
    outs = (yf, yb, hf, cf, hb, cb)
    sum((o.float() * w).sum() for o, w in zip(outs, wts)).backward()
    gemm.check_status()
    got = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    yfr, hfr, cfr = L.lstm_reference(x, lens, *fw, states[0], states[1], reverse=False)
    ybr, hbr, cbr = L.lstm_reference(x, lens, *bw, states[2], states[3], reverse=True)
    sum((o * w).sum() for o, w in zip((yfr, ybr, hfr, cfr, hbr, cbr), wts)).backward()
    for o, r in zip(outs, (yfr, ybr, hfr, cfr, hbr, cbr)):
        torch.testing.assert_close(o.float(), r, atol=0.05, rtol=0.03)
    for g, t in zip(got, leaves):
        scale = float(t.grad.abs().max()) + 1e-6
        assert float((g.float() - t.grad).abs().max()) / scale < 0.06
    # one direction alone takes the same route
    y, h, c = L.lstm(x, lens, *fw, states[0], states[1], reverse=True)
    yr, hr, cr = L.lstm_reference(x, lens, *fw, states[0], states[1], reverse=True)
    torch.testing.assert_close(y.float(), yr, atol=0.05, rtol=0.03)
    torch.testing.assert_close(c.float(), cr, atol=0.05, rtol=0.03)


@gpu
@pytest.mark.parametrize("T,B,I,H", [(20, 10, 32, 100), (15, 60, 64, 320)])
def test_lstm_hidden_sizes_off_the_kernel_grid_run_zero_padded(T, B, I, H):
    """hidden sizes that are not multiples of 128 go through the persistent kernels zero-padded: same function and gradients"""
    from returnn_b200.ops import lstm as L, gemm

    torch.manual_seed(4)
    dev = "cuda"
    x = (torch.randn(T, B, I, device=dev) * 0.5).requires_grad_(True)

    def params():
        return [(torch.randn(4 * H, I, device=dev) * 0.2).requires_grad_(True), (torch.randn(4 * H, H, device=dev) * 0.15).requires_grad_(True),
                (torch.randn(4 * H, device=dev) * 0.1).requires_grad_(True)]

    fw, bw = params(), params()
    states = [(torch.randn(B, H, device=dev) * 0.3).requires_grad_(True) for _ in range(4)]
    lens = torch.sort(torch.randint(1, T + 1, (B,)), descending=True).values
    lens[0] = T
    assert L._padded_hidden(x, fw[1]) == -(-H // 128) * 128
    wts = [torch.randn(T, B, H, device=dev) for _ in range(2)] + [torch.randn(B, H, device=dev) for _ in range(4)]
    leaves = [x] + fw + bw + states
    (yf, hf, cf), (yb, hb, cb) = L.blstm(x, lens, tuple(fw), tuple(bw), *states)
    outs = (yf, yb, hf, cf, hb, cb)
    assert yf.shape == (T, B, H) and cf.shape == (B, H)
    sum((o.float() * w).sum() for o, w in zip(outs, wts)).backward()
    gemm.check_status()
    got = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    yfr, hfr, cfr = L.lstm_reference(x, lens, *fw, states[0], states[1], reverse=False)
    ybr, hbr, cbr = L.lstm_reference(x, lens, *bw, states[2], states[3], reverse=True)
    sum((o * w).sum() for o, w in zip((yfr, ybr, hfr, cfr, hbr, cbr), wts)).backward()
    for o, r in zip(outs, (yfr, ybr, hfr, cfr, hbr, cbr)):
        torch.testing.assert_close(o.float(), r, atol=0.05, rtol=0.03)
    for g, t in zip(got, leaves):
        scale = float(t.grad.abs().max()) + 1e-6
        assert float((g.float() - t.grad).abs().max()) / scale < 0.06
    y, h, c = L.lstm(x, lens, *fw, states[0], states[1])
    torch.testing.assert_close(y.float(), yfr, atol=0.05, rtol=0.03)


@gpu
def test_lstm_input_width_off_the_pitch_rule_and_training_through_the_fallback():
    """9 input features (the 12AX task): the native path takes them zero-padded to 16; gradients flow, also through the cuDNN fallback (hidden 20)"""
    from returnn_b200.ops import lstm as L

    torch.manual_seed(6)
    dev = "cuda"
    for H in (128, 20):
        T, B, I = 11, 4, 9
        x = (torch.randn(T, B, I, device=dev) * 0.5).requires_grad_(True)
        w_ff = (torch.randn(4 * H, I, device=dev) * 0.2).requires_grad_(True)
        w_rec = (torch.randn(4 * H, H, device=dev) * 0.2).requires_grad_(True)
        bias = (torch.randn(4 * H, device=dev) * 0.1).requires_grad_(True)
        h0, c0 = torch.zeros(B, H, device=dev), torch.zeros(B, H, device=dev)
        lens = torch.tensor([11, 7, 11, 2])
        y, h, c = L.lstm(x, lens, w_ff, w_rec, bias, h0, c0)
        y.float().square().sum().backward()
        got = [t.grad.clone() for t in (x, w_ff, w_rec, bias)]
        for t in (x, w_ff, w_rec, bias):
            t.grad = None
        yr, hr, cr = L.lstm_reference(x, lens, w_ff, w_rec, bias, h0, c0)
        yr.square().sum().backward()
        torch.testing.assert_close(y.float(), yr, atol=0.05, rtol=0.03)
        for g, t in zip(got, (x, w_ff, w_rec, bias)):
            assert float((g.float() - t.grad).abs().max()) / (float(t.grad.abs().max()) + 1e-6) < 0.06
