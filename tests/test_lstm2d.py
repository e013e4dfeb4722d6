"""2-D LSTM (returnn_b200/ops/lstm2d.py): the diagonal-wise implementation against a cell-by-cell autograd restatement."""

import pytest
import torch

gpu = pytest.mark.gpu


def _check(dev, dtype=torch.float64, atol=1e-9):
    from returnn_b200.ops import lstm2d

    torch.manual_seed(0)
    T, S, B, n_in, n = 4, 5, 3, 6, 7
    mk = lambda *shape: (torch.randn(*shape, dtype=dtype, device=dev) * 0.4).requires_grad_(True)  # noqa: E731
    x, w, v_h, v_v, b = mk(T, S, B, n_in), mk(n_in, 5 * n), mk(n, 5 * n), mk(n, 5 * n), mk(5 * n)
    sizes = torch.tensor([[4, 5], [2, 3], [3, 1]], device=dev)
    gy, gc = torch.randn(T, S, B, n, dtype=dtype, device=dev), torch.randn(T, S, B, n, dtype=dtype, device=dev)
    for sz in (None, sizes):
        for p in (x, w, v_h, v_v, b):
            p.grad = None
        h, c = lstm2d.two_d_lstm(x, w, v_h, v_v, b, sz)
        ((h * gy).sum() + (c * gc).sum()).backward()
        got = [p.grad.clone() for p in (x, w, v_h, v_v, b)]
        for p in (x, w, v_h, v_v, b):
            p.grad = None
        h_ref, c_ref = lstm2d.two_d_lstm_reference(x, w, v_h, v_v, b, sz)
        ((h_ref * gy).sum() + (c_ref * gc).sum()).backward()
        torch.testing.assert_close(h.to(dtype), h_ref, atol=atol, rtol=0)
        torch.testing.assert_close(c.to(dtype), c_ref, atol=atol, rtol=0)
        for g, p, name in zip(got, (x, w, v_h, v_v, b), ("x", "w", "v_h", "v_v", "b")):
            torch.testing.assert_close(g, p.grad, atol=atol * 10, rtol=0, msg=lambda m, name=name: "grad of %s: %s" % (name, m))
        if sz is not None:
            assert float(h[2:, :, 1].abs().max()) == 0.0 and float(h[:, 3:, 1].abs().max()) == 0.0 and float(x.grad[3, 2, 2].abs().max()) == 0.0


def test_two_d_lstm_cpu():
    _check("cpu", torch.float32, atol=2e-5)


@gpu
def test_two_d_lstm_cell_kernels():
    _check("cuda", torch.float32, atol=5e-5)
