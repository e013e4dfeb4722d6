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
