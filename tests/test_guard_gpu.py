"""
Out-of-bounds and stream-order checks of the native kernels on ragged shapes (ops/guard.py): every tensor a wrapper allocates
sits between canary regions; forward and backward run; afterwards no canary may be damaged. A second pass runs ops under a
delayed-stream schedule and twice on the same inputs.
"""

import pytest
import torch

gpu = pytest.mark.gpu


def _need_lib():
    from returnn_b200.ops import _lib

    if _lib.get_lib() is None:
        pytest.fail("native library missing on a GPU machine")


def _run_guarded(fn):
    from returnn_b200.ops import guard, gemm

    with guard.CanaryAllocations() as g:
        res = fn()
        outs = [t for t in guard._flatten(res) if t.requires_grad]
        if outs:
            sum((t.float() * torch.linspace(-1, 1, t.numel(), device=t.device).view(t.shape)).sum() for t in outs).backward()
    g.check()
    gemm.check_status()
    assert g.num_guarded() > 0, "no allocation of the op went through the guard: the native path did not run"
    return res


@gpu
@pytest.mark.parametrize("rows,n", [(1, 512), (37, 512), (1001, 384), (3, 2048), (130, 40)])
def test_layer_norm_and_rms_norm_stay_in_bounds(rows, n):
    _need_lib()
    from returnn_b200.ops import layer_norm as ln

    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(rows, n, device="cuda", dtype=dtype, requires_grad=True)
        gamma = torch.randn(n, device="cuda", requires_grad=True)
        beta = torch.randn(n, device="cuda", requires_grad=True)
        _run_guarded(lambda: ln.layer_norm(x, gamma, beta, 1e-5))
        _run_guarded(lambda: ln.rms_norm(x, gamma, None, 1e-5))


@gpu
@pytest.mark.parametrize("m,k,n", [(1, 64, 64), (77, 512, 520), (1000, 72, 2048), (4097, 512, 8), (130, 2048, 512)])
def test_linear_gemm_stays_in_bounds(m, k, n):
    _need_lib()
    from returnn_b200.ops import linear as L

    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(k, n, device="cuda") * 0.05).requires_grad_(True)
    b = torch.randn(n, device="cuda", requires_grad=True)
    for act in (None, "relu", "silu"):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _run_guarded(lambda: L.linear(x, w, b, act))


@gpu
@pytest.mark.parametrize("rows,v", [(1, 8), (5, 10001), (33, 32000), (7, 13)])
def test_softmax_ce_and_dropout_stay_in_bounds(rows, v):
    _need_lib()
    from returnn_b200.ops import softmax_ce as ce, elementwise as ew

    for dtype in (torch.bfloat16, torch.float32):
        logits = torch.randn(rows, v, device="cuda", dtype=dtype, requires_grad=True)
        tgt = torch.randint(0, v, (rows,), device="cuda", dtype=torch.int32)
        _run_guarded(lambda: ce.softmax_cross_entropy(logits, tgt, 0.1))
        _run_guarded(lambda: ce.softmax_cross_entropy(logits, tgt, 0.1, grad_only_smoothing=True, with_argmax=True)[0])
    x = torch.randn(rows, v, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    _run_guarded(lambda: ew.dropout(x, 0.3))


@gpu
@pytest.mark.parametrize("B,Tq,Tk,H,D", [(1, 1, 1, 1, 64), (3, 37, 53, 4, 64), (2, 65, 64, 2, 128), (5, 128, 7, 8, 64)])
def test_sdpa_stays_in_bounds(B, Tq, Tk, H, D):
    _need_lib()
    from returnn_b200.ops import sdpa as S

    q = torch.randn(B, Tq, H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, Tk, H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, Tk, H * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    lens = torch.randint(1, Tk + 1, (B,), dtype=torch.int32)
    assert S.supports(q, k, H)
    _run_guarded(lambda: S.sdpa(q, k, v, num_heads=H, k_lens=lens, causal=False, dropout_p=0.1))
    if Tq <= Tk:
        _run_guarded(lambda: S.sdpa(q, k, v, num_heads=H, k_lens=None, causal=True))


@gpu
@pytest.mark.parametrize("T,B,I,H", [(1, 1, 8, 128), (9, 5, 16, 32), (23, 48, 64, 128), (17, 49, 32, 128), (11, 7, 24, 256)])
def test_lstm_and_blstm_stay_in_bounds(T, B, I, H):
    _need_lib()
    from returnn_b200.ops import lstm as L

    x = (torch.randn(T, B, I, device="cuda") * 0.5).requires_grad_(True)
    ps = [[(torch.randn(4 * H, I, device="cuda") * 0.2).requires_grad_(True), (torch.randn(4 * H, H, device="cuda") * 0.1).requires_grad_(True),
           torch.zeros(4 * H, device="cuda", requires_grad=True)] for _ in range(2)]
    st = [torch.zeros(B, H, device="cuda") for _ in range(4)]
    lens = torch.randint(1, T + 1, (B,), dtype=torch.int32)
    lens[0] = T
    _run_guarded(lambda: L.lstm(x, lens, *ps[0], st[0], st[1], reverse=True)[0])

    def both():
        (yf, _, _), (yb, _, _) = L.blstm(x, lens, tuple(ps[0]), tuple(ps[1]), *st)
        return yf, yb

    _run_guarded(both)


@gpu
def test_ctc_stays_in_bounds():
    _need_lib()
    from returnn_b200.ops import ctc

    for B, T, V, S in ((1, 1, 9, 1), (3, 50, 10001, 17), (6, 33, 41, 16)):
        logits = torch.randn(B, T, V, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        tl = torch.randint(1, S + 1, (B,), dtype=torch.int32)
        il = torch.full((B,), T, dtype=torch.int32)
        il[-1] = max(1, T - 3)
        tl = torch.minimum(tl, (il // 2).clamp(min=1))
        targets = torch.randint(0, V - 1, (B, int(tl.max())), device="cuda", dtype=torch.int32)
        if not ctc.supports(logits, targets):
            continue
        _run_guarded(lambda: ctc.ctc_loss(logits, targets, il, tl, blank_index=V - 1))


@gpu
def test_kernels_respect_the_current_stream_and_are_repeatable():
    """delayed producer stream + side stream against the default stream; same inputs twice"""
    _need_lib()
    from returnn_b200.ops import guard, layer_norm as ln, linear as L, softmax_ce as ce, sdpa as S

    gen = lambda *shape: torch.randn(*shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
    gamma, beta = torch.ones(512, device="cuda"), torch.zeros(512, device="cuda")
    guard.check_stream_order(lambda: [gen(301, 512).to(torch.bfloat16)], lambda x: ln.layer_norm(x, gamma, beta, 1e-5))
    w, b = gen(512, 1024) * 0.05, gen(1024)

    def lin(x):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return L.linear(x, w, b, "relu")

    guard.check_stream_order(lambda: [gen(777, 512).to(torch.bfloat16)], lin)
    tgt = torch.randint(0, 10001, (64,), device="cuda", dtype=torch.int32)
    guard.check_stream_order(lambda: [gen(64, 10001).to(torch.bfloat16)], lambda z: ce.softmax_cross_entropy(z, tgt, 0.1))
    guard.check_stream_order(lambda: [gen(2, 40, 256).to(torch.bfloat16), gen(2, 50, 256).to(torch.bfloat16)],
                             lambda q, k: S.sdpa(q, k, k, num_heads=4))
    x = gen(301, 512).to(torch.bfloat16)
    guard.check_repeatable(lambda: ln.layer_norm(x, gamma, beta, 1e-5))
    guard.check_repeatable(lambda: lin(x))
