"""Sequence utility ops: CPU references against brute force, and the B200 kernels against the references."""

import pytest
import torch

gpu = pytest.mark.gpu


def _ed_data(dev):
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 6, (9, 40), generator=g)
    b = torch.randint(0, 6, (9, 70), generator=g)
    al = torch.tensor([40, 1, 0, 17, 33, 5, 40, 2, 39])
    bl = torch.tensor([70, 0, 3, 17, 64, 70, 1, 2, 33])
    b[3, :17] = a[3, :17]
    return a.to(dev), al, b.to(dev), bl


def test_edit_distance_reference_known_cases():
    from returnn_b200.ops import seq_ops

    a = torch.tensor([[1, 2, 3, 4], [1, 2, 3, 4]])
    b = torch.tensor([[1, 3, 4, 0], [5, 6, 7, 8]])
    d = seq_ops.edit_distance(a, torch.tensor([4, 4]), b, torch.tensor([3, 4]))
    assert d.tolist() == [1, 4]


def test_rnnt_reference_matches_brute_force():
    from returnn_b200.ops import seq_ops
    import itertools, math

    torch.manual_seed(0)
    T, U = 3, 2
    lp = torch.log_softmax(torch.randn(1, T, U + 1, 2), dim=-1)
    loss = seq_ops.rnnt_loss(lp[..., 0], lp[..., 1], torch.tensor([T]), torch.tensor([U]))
    # all monotonic paths: sequences of T blanks and U labels ending with a blank
    total = -math.inf
    for pos in itertools.combinations(range(T + U - 1), U):
        t = u = 0
        s = 0.0
        for step in range(T + U - 1):
            if step in pos:
                s += float(lp[0, t, u, 1]); u += 1
            else:
                s += float(lp[0, t, u, 0]); t += 1
        s += float(lp[0, T - 1, U, 0])
        total = max(total, s) + math.log1p(math.exp(-abs(total - s))) if total > -math.inf else s
    assert abs(float(loss) + total) < 1e-4


def test_beam_topk_reference_finished_hyps():
    from returnn_b200.ops import seq_ops

    logits = torch.zeros(1, 2, 4)
    logits[0, 0, 2] = 5.0
    prev = torch.tensor([[0.0, -0.1]])
    fin = torch.tensor([[False, True]])
    s, back, lab = seq_ops.beam_topk(logits, prev, finished=fin, eos=3, k=2)
    assert back.tolist() == [[0, 1]] and lab.tolist() == [[2, 3]] and abs(float(s[0, 1]) + 0.1) < 1e-6


@gpu
def test_edit_distance_kernel():
    from returnn_b200.ops import seq_ops

    a, al, b, bl = _ed_data("cuda")
    got = seq_ops.edit_distance(a, al, b, bl)
    ref = seq_ops.edit_distance_reference(a.cpu(), al, b.cpu(), bl)
    assert got.cpu().tolist() == ref.tolist()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("k,beam,V", [(12, 12, 10001), (4, 1, 57), (32, 8, 1000), (8, 40, 501), (16, 64, 33)])
def test_beam_topk_kernel(dtype, k, beam, V):
    from returnn_b200.ops import seq_ops

    torch.manual_seed(1)
    logits = (torch.randn(5, beam, V, device="cuda") * 3).to(dtype)
    prev = torch.randn(5, beam, device="cuda")
    fin = torch.rand(5, beam, device="cuda") < 0.2
    s, back, lab = seq_ops.beam_topk(logits, prev, finished=fin, eos=3, k=k)
    rs, rback, rlab = seq_ops.beam_topk_reference(logits, prev, fin, 3, k)
    torch.testing.assert_close(s, rs, atol=2e-3, rtol=1e-4)
    # indices may differ only where scores tie
    same = (back == rback) & (lab == rlab)
    assert bool((same | ((s - rs).abs() < 2e-3)).all())
    assert float(same.float().mean()) > 0.9


@gpu
def test_rnnt_kernel_loss_and_grad():
    from returnn_b200.ops import seq_ops

    torch.manual_seed(2)
    B, T, U, V = 3, 11, 5, 7
    joint = torch.randn(B, T, U + 1, V, device="cuda", requires_grad=True)
    targets = torch.randint(1, V, (B, U), device="cuda")
    t_lens, u_lens = torch.tensor([11, 7, 1]), torch.tensor([5, 2, 0])
    loss = seq_ops.rnnt_loss_from_joint(joint, targets, t_lens, u_lens)
    loss.sum().backward()
    g = joint.grad.clone()
    joint2 = joint.detach().cpu().requires_grad_(True)
    ref = seq_ops.rnnt_loss_from_joint(joint2, targets.cpu(), t_lens, u_lens)
    ref.sum().backward()
    torch.testing.assert_close(loss.cpu(), ref, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(g.cpu(), joint2.grad, atol=1e-3, rtol=1e-3)


@gpu
def test_device_assert_records_failure_without_trap():
    from returnn_b200.ops import seq_ops

    x = torch.arange(100, device="cuda")
    seq_ops.device_assert(x >= 0, "all non-negative")
    seq_ops.check_asserts()
    seq_ops.device_assert(x != 37, "no 37 allowed")
    with pytest.raises(AssertionError, match="no 37 allowed.*element 37"):
        seq_ops.check_asserts()
    # the context is still usable
    assert int((x + 1).sum()) == 5050


def _seq_util_checks(dev):
    from returnn_b200.ops import seq_util as su

    torch.manual_seed(0)
    T, B, D = 11, 3, 4
    x = torch.randn(T, B, D, device=dev)
    lens = torch.tensor([11, 7, 4])
    for b in range(B):
        x[int(lens[b]):, b] = 0
    y, ym = su.chunk(x, lens, chunk_size=5, chunk_step=3)
    n = su.num_chunks(T, 5, 3)
    assert n == 3 and tuple(y.shape) == (5, B * n, D) and tuple(ym.shape) == (5, B * n)
    for b in range(B):
        for c in range(n):
            for ot in range(5):
                t = c * 3 + ot
                ok = t < int(lens[b])
                assert float(ym[ot, b * n + c]) == float(ok)
                assert torch.equal(y[ot, b * n + c], x[t, b] if ok else torch.zeros(D, device=dev))
    back, bm, fac = su.unchunk(y, ym, T=T, B=B, chunk_size=5, chunk_step=3)
    torch.testing.assert_close(back, x, atol=1e-6, rtol=0)  # the mean of equal copies is the value itself
    assert torch.equal(bm, (torch.arange(T, device=dev)[:, None] < lens.to(dev)[None, :]).float())
    assert float(fac[3, 0]) == 0.5 and float(fac[0, 0]) == 1.0 and float(fac[5, 0]) == 1.0  # frames 3, 4 lie in windows 0 and 1
    # windows with different content: overlap is averaged
    y2 = y.clone()
    y2[3, 0 * n + 0] += 2.0  # frame 3 of sequence 0 as seen by window 0
    back2, _, _ = su.unchunk(y2, ym, T=T, B=B, chunk_size=5, chunk_step=3)
    torch.testing.assert_close(back2[3, 0], x[3, 0] + 1.0, atol=1e-6, rtol=0)
    # select by index
    xs = torch.randn(T, B, D, device=dev, requires_grad=True)
    idx = torch.randint(0, D, (T, B), device=dev)
    sel = su.select_by_index(xs, idx)
    torch.testing.assert_close(sel, torch.gather(xs, -1, idx[..., None]).squeeze(-1))
    gy = torch.randn(T, B, device=dev)
    sel.backward(gy)
    ref = torch.zeros(T, B, D, device=dev).scatter_(-1, idx[..., None], gy[..., None])
    torch.testing.assert_close(xs.grad, ref)
    # COO targets
    n_e = 9
    s0 = torch.randint(0, T, (n_e, B), device=dev)
    s1 = torch.randint(0, D, (n_e, B), device=dev)
    w = torch.rand(n_e, B, device=dev)
    m = (torch.rand(n_e, B, device=dev) > 0.2).float()
    dense = su.sparse_to_dense(s0, s1, w, m, T=T, D=D)
    ref = torch.zeros(T, B, D, device=dev)
    for i in range(n_e):
        for b in range(B):
            if m[i, b] > 0:
                ref[s0[i, b], b, s1[i, b]] += w[i, b]
    torch.testing.assert_close(dense, ref)
    mx, am = su.max_and_argmax_sparse(s0, s1, w, m, T=T)
    for t in range(T):
        for b in range(B):
            ent = [(float(w[i, b]), int(s1[i, b])) for i in range(n_e) if m[i, b] > 0 and int(s0[i, b]) == t]
            if ent:
                best = max(ent, key=lambda e: (e[0], -e[1]))
                assert abs(float(mx[t, b]) - best[0]) < 1e-7 and int(am[t, b]) == best[1]
            else:
                assert float(mx[t, b]) == float("-inf")
    z = torch.randn(T, B, D, device=dev)
    zm = (torch.arange(T, device=dev)[:, None] < lens.to(dev)[None, :]).float()
    ce, g = su.sparse_ce_softmax_and_grad(z, zm, s0, s1, w, m)
    logp = torch.log_softmax(z, -1)
    torch.testing.assert_close(ce, -(ref * logp).sum(-1) * zm, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(g, (logp.exp() - ref) * zm[..., None], atol=1e-5, rtol=1e-5)


def test_seq_util_references_cpu():
    _seq_util_checks("cpu")


@gpu
def test_seq_util_kernels():
    _seq_util_checks("cuda")


def _levenshtein_row(a, b):
    """distances of a to every prefix of b"""
    row = list(range(len(b) + 1))
    for i, x in enumerate(a):
        new = [i + 1]
        for j, y in enumerate(b):
            new.append(min(row[j + 1] + 1, new[j] + 1, row[j] + (x != y)))
        row = new
    return row


def test_row_wise_edit_distance_family():
    """next_edit_distance_row / _reduce and the optimal-completion forms against a plain dynamic program"""
    import torch
    from returnn_b200.torch.util import native_op as N

    g = torch.Generator().manual_seed(5)
    B, t1, t2, V = 6, 7, 9, 4
    a = torch.randint(0, V, (B, t1), generator=g, dtype=torch.int32)
    b = torch.randint(0, V, (B, t2), generator=g, dtype=torch.int32)
    a_len = torch.tensor([7, 3, 0, 5, 7, 1], dtype=torch.int32)
    b_len = torch.tensor([9, 4, 6, 0, 2, 9], dtype=torch.int32)
    full = N.edit_distance_via_next_edit_distance_row(a, a_len, b, b_len, full_row_output=True)
    for i in range(B):
        want = _levenshtein_row(a[i, : a_len[i]].tolist(), b[i, : b_len[i]].tolist())
        assert full[i, : b_len[i] + 1].tolist() == want
        assert full[i, b_len[i]:].tolist() == [want[-1]] * (t2 + 1 - int(b_len[i]))  # the entry at b_len is repeated
    dist = N.edit_distance_via_next_edit_distance_row(a, a_len, b, b_len)
    assert dist.tolist() == N.edit_distance(a, a_len, b, b_len).tolist()
    oc = N.optimal_completion_edit_distance(a, a_len, b, b_len)
    assert oc.tolist() == [min(_levenshtein_row(a[i, : a_len[i]].tolist(), b[i, : b_len[i]].tolist())) for i in range(B)]
    per = N.optimal_completion_edit_distance_per_successor(a, a_len, b, b_len, V)
    assert per.shape == (B, V)
    for i in range(B):
        for s in range(V):
            assert int(per[i, s]) == min(_levenshtein_row(a[i, : a_len[i]].tolist() + [s], b[i, : b_len[i]].tolist()))
    # the loop form: sequences of full length are extended, shorter ones count as ended (their row is kept)
    via = N.optimal_completion_edit_distance_per_successor_via_next_edit_distance(a, a_len, b, b_len, V)
    for i in range(B):
        for s in range(V):
            ext = a[i, : a_len[i]].tolist() + ([s] if int(a_len[i]) == t1 else [])
            assert int(via[i, s]) == min(_levenshtein_row(ext, b[i, : b_len[i]].tolist()))
    # a blank candidate keeps the row
    row = N.edit_distance_via_next_edit_distance_row(a, a_len, b, b_len, full_row_output=True)
    red = N.next_edit_distance_reduce(row, torch.arange(V)[None], torch.tensor(t1), torch.zeros(B, dtype=torch.bool), b, b_len, a_blank_idx=2)
    assert red[:, 2].tolist() == row[:, -1].tolist()
    assert N.make_op("EditDistanceOp") is N.edit_distance and N.make_fast_baum_welch_op() is N.fast_baum_welch


def test_ctc_best_path_facade():
    import torch
    from returnn_b200.torch.util import native_op as N

    torch.manual_seed(0)
    logits = torch.randn(2, 8, 5)
    tl = torch.tensor([3, 2], dtype=torch.int32)
    il = torch.tensor([8, 5], dtype=torch.int32)
    y = torch.tensor([[1, 2, 1], [3, 3, 0]], dtype=torch.int32)
    p = N.ctc_best_path(logits=logits, logits_seq_lens=il, targets=y, targets_seq_lens=tl, blank_index=4)
    assert p.shape == (2, 8) and p[1, 5:].tolist() == [4, 4, 4]
    for i in range(2):
        path = p[i, : il[i]].tolist()
        collapsed = [v for k, v in enumerate(path) if v != 4 and (k == 0 or v != path[k - 1])]
        assert collapsed == y[i, : tl[i]].tolist()
