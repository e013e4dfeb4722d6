"""FSA ops: CTC via the FSA full sum equals torch's CTC loss (values and gradients); Viterbi equals the brute-force best path."""

import pytest
import torch

gpu = pytest.mark.gpu


def _case(dev, B=4, T=13, V=6, S=4):
    torch.manual_seed(0)
    logits = torch.randn(B, T, V, device=dev, requires_grad=True)
    targets = torch.randint(0, V - 1, (B, S), device=dev)
    targets[1, 1] = targets[1, 0]  # a repeated label needs the blank in between
    in_lens = torch.tensor([13, 9, 13, 5])[:B]
    tgt_lens = torch.tensor([4, 3, 0, 2])[:B]
    return logits, targets, in_lens, tgt_lens


def _check(dev):
    from returnn_b200.ops import fsa

    logits, targets, in_lens, tgt_lens = _case(dev)
    V = logits.shape[-1]
    loss = fsa.ctc_loss_via_fsa(logits, targets, in_lens, tgt_lens, blank=V - 1)
    loss.sum().backward()
    g = logits.grad.clone()
    l2 = logits.detach().cpu().requires_grad_(True)
    ref = torch.nn.functional.ctc_loss(torch.log_softmax(l2, -1).transpose(0, 1), targets.cpu(), in_lens, tgt_lens, blank=V - 1, reduction="none")
    ref.sum().backward()
    torch.testing.assert_close(loss.cpu(), ref, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(g.cpu(), l2.grad, atol=1e-3, rtol=1e-3)
    # Viterbi: its score is at least as good as any sampled alignment and equals the greedy path when that path is valid
    f = fsa.ctc_fsa(targets, tgt_lens, blank=V - 1)
    am = -torch.log_softmax(logits.detach().float(), -1).transpose(0, 1).contiguous()
    align, score = fsa.fast_viterbi(am, f, in_lens)
    align_ref, score_ref = fsa.fast_viterbi_reference(am.cpu(), f.to("cpu"), in_lens)
    torch.testing.assert_close(score.cpu(), score_ref, atol=1e-3, rtol=1e-4)
    for b in range(logits.shape[0]):
        path = align[: int(in_lens[b]), b].cpu().tolist()
        collapsed = [p for i, p in enumerate(path) if p != V - 1 and (i == 0 or p != path[i - 1])]
        assert collapsed == targets[b, : int(tgt_lens[b])].cpu().tolist()
        assert abs(float(am[: int(in_lens[b]), b].cpu().gather(1, torch.tensor(path)[:, None]).sum()) - float(score[b])) < 1e-3


def test_ctc_via_fsa_cpu():
    _check("cpu")


@gpu
def test_ctc_via_fsa_kernels():
    _check("cuda")


def _multi_end_case(dev):
    """two sequences over a 3-state left-to-right chain (loop + forward edges); several weighted final states"""
    from returnn_b200.ops.fsa import FsaBatch

    torch.manual_seed(3)
    T, B, V = 6, 2, 4
    am = torch.rand(T, B, V, device=dev) * 2.0
    ef, et, ee, ww, estart = [], [], [], [], [0]
    for b in range(B):
        base = 3 * b
        for s in range(3):
            ef.append(base + s); et.append(base + s); ee.append(s); ww.append(0.1 * (s + 1))
            if s < 2:
                ef.append(base + s); et.append(base + s + 1); ee.append(s + 1); ww.append(0.3)
        estart.append(len(ef))
    mk = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt, device=dev)  # noqa: E731
    f = FsaBatch(mk(ef), mk(et), mk(ee), mk(ww, torch.float32), mk(estart), mk([0, 3]), mk([2, 5]), mk([-1, -1]), 6)
    lens = torch.tensor([6, 4])
    end_states = torch.tensor([[1, 5], [0, 2], [0, 1], [1, 4]])  # unsorted on purpose
    end_weights = torch.tensor([0.0, 0.2, 1.5, 0.7])
    return am, f, lens, end_states, end_weights


def _brute_force_paths(am, f, b, Tb, ends):
    """-log of the sum over all paths of sequence b, and the -log posterior per (t, label), by enumeration"""
    import itertools, math

    ef, et, ee, ww = f.e_from.tolist(), f.e_to.tolist(), f.e_em.tolist(), f.weights.tolist()
    e0, e1 = int(f.edge_start[b]), int(f.edge_start[b + 1])
    total = 0.0
    V = am.shape[2]
    occ = [[0.0] * V for _ in range(Tb)]
    for path in itertools.product(range(e0, e1), repeat=Tb):
        st = int(f.start[b])
        cost = 0.0
        ok = True
        for t, e in enumerate(path):
            if ef[e] != st:
                ok = False
                break
            cost += ww[e] + float(am[t, b, ee[e]])
            st = et[e]
        if not ok or st not in ends:
            continue
        p = math.exp(-cost - ends[st])
        total += p
        for t, e in enumerate(path):
            occ[t][ee[e]] += p
    return total, occ


def _check_multi_end(dev):
    import math
    from returnn_b200.ops import fsa

    am, f, lens, end_states, end_weights = _multi_end_case(dev)
    out, obs = fsa.fast_baum_welch_multi_end(am, f, lens, end_states=end_states, end_state_weights=end_weights)
    for b in range(2):
        ends = {int(s): float(w) for (q, s), w in zip(end_states.tolist(), end_weights.tolist()) if q == b}
        total, occ = _brute_force_paths(am.cpu(), f.to("cpu"), b, int(lens[b]), ends)
        assert abs(float(obs[b]) + math.log(total)) < 1e-4
        for t in range(int(lens[b])):
            for v in range(am.shape[2]):
                got = math.exp(-float(out[t, b, v]))
                assert abs(got - occ[t][v] / total) < 1e-4, (b, t, v, got, occ[t][v] / total)
    # a single final state of weight 0 per sequence is the plain op
    single = torch.tensor([[0, 2], [1, 5]])
    out1, obs1 = fsa.fast_baum_welch_multi_end(am, f, lens, end_states=single, end_state_weights=torch.zeros(2))
    out2, obs2 = fsa.fast_baum_welch(am, f, lens)
    torch.testing.assert_close(obs1.cpu(), obs2.cpu(), atol=1e-4, rtol=1e-5)
    fin = torch.isfinite(out2.cpu())
    assert bool((torch.isfinite(out1.cpu()) == fin).all())
    torch.testing.assert_close(out1.cpu()[fin], out2.cpu()[fin], atol=1e-4, rtol=1e-5)


def test_multi_end_baum_welch_cpu():
    _check_multi_end("cpu")


@gpu
def test_multi_end_baum_welch_kernel():
    _check_multi_end("cuda")


def _segment_case(dev):
    from returnn_b200.ops.fsa import FsaBatch

    torch.manual_seed(4)
    B, L, V = 2, 3, 3
    lens = torch.tensor([5, 4])
    row_start = torch.tensor([0, 5])
    N = 9
    am = torch.rand(N, L, V, device=dev) * 2.0
    length_models = torch.tensor([[0.2, 0.9, 1.6], [1.1, 0.4, 0.8]], device=dev)
    # per sequence: states 0 -> 1 -> 2 (labels 0, 1, 2 on the forward edges), plus a loop on the middle state with label 1
    ef, et, ee, ww, lm, estart = [], [], [], [], [], [0]
    for b in range(B):
        base = 3 * b
        for (a, c, lab, w, m) in ((0, 1, 0, 0.1, 0), (1, 1, 1, 0.5, 1), (1, 2, 2, 0.2, 0), (0, 2, 2, 1.0, 1)):
            ef.append(base + a); et.append(base + c); ee.append(lab); ww.append(w); lm.append(m)
        estart.append(len(ef))
    mk = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt, device=dev)  # noqa: E731
    f = FsaBatch(mk(ef), mk(et), mk(ee), mk(ww, torch.float32), mk(estart), mk([0, 3]), mk([2, 5]), mk([-1, -1]), 6)
    return am, f, mk(lm), length_models, row_start, lens


def _check_segment(dev):
    import math
    from returnn_b200.ops import fsa

    am, f, lm, length_models, row_start, lens = _segment_case(dev)
    scale = 0.7
    out, obs = fsa.segment_fast_baum_welch(am, f, e_lenmod=lm, length_models=length_models, row_start=row_start, lens=lens, am_scale=scale)
    N, L, V = am.shape
    amc, lmc = am.cpu(), length_models.cpu()
    ef, et, ee, ww, lml = f.e_from.tolist(), f.e_to.tolist(), f.e_em.tolist(), f.weights.tolist(), lm.tolist()
    for b in range(2):
        Tb, r0 = int(lens[b]), int(row_start[b])
        e0, e1 = int(f.edge_start[b]), int(f.edge_start[b + 1])
        total = 0.0
        occ = {}

        def walk(t, st, cost, segs):
            nonlocal total
            if t == Tb:
                if st == int(f.end[b]):
                    p = math.exp(-cost)
                    total += p
                    for key in segs:
                        occ[key] = occ.get(key, 0.0) + p
                return
            for e in range(e0, e1):
                if ef[e] != st:
                    continue
                for l in range(min(L, Tb - t)):
                    c = ww[e] + scale * float(amc[r0 + t, l, ee[e]]) + float(lmc[lml[e], l])
                    walk(t + l + 1, et[e], cost + c, segs + [(r0 + t, l, ee[e])])

        walk(0, int(f.start[b]), 0.0, [])
        assert total > 0 and abs(float(obs[b]) + math.log(total)) < 1e-4
        for n in range(r0, r0 + Tb):
            for l in range(L):
                for v in range(V):
                    got = math.exp(-float(out[n, l, v]))
                    assert abs(got - occ.get((n, l, v), 0.0) / total) < 1e-4, (b, n, l, v)


def test_segment_baum_welch_cpu():
    _check_segment("cpu")


@gpu
def test_segment_baum_welch_kernel():
    _check_segment("cuda")


def _check_packed(dev):
    from returnn_b200.ops import fsa

    logits, targets, in_lens, tgt_lens = _case(dev)
    V = logits.shape[-1]
    f = fsa.ctc_fsa(targets, tgt_lens, blank=V - 1)
    am = -torch.log_softmax(logits.detach().float(), -1).transpose(0, 1).contiguous()  # [T, B, V]
    out_ref, obs_ref = fsa.fast_baum_welch(am, f, in_lens)
    rows = [am[: int(in_lens[b]), b] for b in range(am.shape[1])]
    packed = torch.cat(rows)
    row_start = torch.tensor([0] + torch.cumsum(in_lens, 0).tolist()[:-1])
    out, obs = fsa.fast_baum_welch_packed(packed, f, row_start=row_start, lens=in_lens)
    torch.testing.assert_close(obs.cpu(), obs_ref.cpu(), atol=1e-4, rtol=1e-5)
    for b in range(am.shape[1]):
        a = out[int(row_start[b]): int(row_start[b]) + int(in_lens[b])].cpu()
        r = out_ref[: int(in_lens[b]), b].cpu()
        fin = torch.isfinite(r)
        assert bool((torch.isfinite(a) == fin).all())
        torch.testing.assert_close(a[fin], r[fin], atol=1e-4, rtol=1e-5)


def test_packed_baum_welch_cpu():
    _check_packed("cpu")


@gpu
def test_packed_baum_welch_kernel():
    _check_packed("cuda")
