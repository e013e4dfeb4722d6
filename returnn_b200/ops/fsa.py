"""
Batched FSA ops: full-sum forward-backward, Viterbi alignment, CTC topology construction (``csrc/fsa.cu``), each with a
vectorised torch reference that is also the CPU path.

An FSA batch is a :class:`FsaBatch`: edge arrays ``from, to, emission`` (int32 ``[E]``, grouped by sequence with
``edge_start [B+1]``), ``weights [E]`` (negative log), ``start / end / end2 [B]`` state indices (``end2 = -1``: only one
final state) and the total number of states. Every edge consumes one frame.

Two generalisations run on the same engine: any number of weighted final states per sequence (``fast_baum_welch_multi_end``;
MultiEndFastBaumWelchOp, returnn/native_op.py:4064) and edges that consume a whole segment of 1 .. L frames with a length model
(``segment_fast_baum_welch``; SegmentFastBaumWelchOp, :4369).

Reference ops: FastBaumWelchOp (returnn/native_op.py:3259), FastViterbiOp (:4948), GetCtcFsaFastBwOp (:5320);
``ctc_loss_via_fsa`` is the counterpart of the ``use_native_op=True`` path of ``rf.ctc_loss``
(returnn/torch/frontend/_backend.py:832-843).
"""

from __future__ import annotations
from dataclasses import dataclass
from typing import Optional, Tuple
import ctypes
import torch
from . import _lib

_vp, _i32 = ctypes.c_void_p, ctypes.c_int


@dataclass
class FsaBatch:
    """edges of B acceptors in one state index space"""

    e_from: torch.Tensor
    e_to: torch.Tensor
    e_em: torch.Tensor
    weights: torch.Tensor
    edge_start: torch.Tensor
    start: torch.Tensor
    end: torch.Tensor
    end2: torch.Tensor
    num_states: int

    def to(self, device) -> "FsaBatch":
        """same FSA on another device"""
        return FsaBatch(*[getattr(self, n).to(device) for n in ("e_from", "e_to", "e_em", "weights", "edge_start", "start", "end", "end2")], self.num_states)

    @property
    def batch(self) -> int:
        """number of sequences"""
        return int(self.start.shape[0])

    def edge_seq(self) -> torch.Tensor:
        """sequence index per edge"""
        counts = self.edge_start[1:] - self.edge_start[:-1]
        return torch.repeat_interleave(torch.arange(self.batch, device=self.e_from.device), counts.long())


def _native(t: torch.Tensor, name: str) -> bool:
    return t.is_cuda and _lib.use_native(t) and hasattr(_lib.get_lib(), name)


def ctc_fsa(targets: torch.Tensor, tgt_lens: torch.Tensor, *, blank: int, label_loop: bool = True) -> FsaBatch:
    """
    CTC topology for every target sequence: ``2*S+1`` states (blank, l1, blank, ..., blank); with ``label_loop=False`` labels
    cannot repeat (RNA-like topology).
    """
    B = targets.shape[0]
    dev = targets.device
    lens = tgt_lens.to(dev).to(torch.int64)
    n_states = 2 * lens + 1
    state_base = torch.zeros(B + 1, dtype=torch.int64, device=dev)
    state_base[1:] = torch.cumsum(n_states, 0)
    edge_start = (3 * state_base).to(torch.int32)
    S_total = int(state_base[-1])
    E = 3 * S_total
    tg = targets.to(torch.int32).contiguous()
    if _native(tg, "rb200_ctc_fsa"):
        e_from = torch.empty(E, dtype=torch.int32, device=dev)
        e_to, e_em = torch.empty_like(e_from), torch.empty_like(e_from)
        w = torch.empty(E, dtype=torch.float32, device=dev)
        start, end, end2 = (torch.empty(B, dtype=torch.int32, device=dev) for _ in range(3))
        sb32, eb32, l32 = state_base[:-1].to(torch.int32).contiguous(), edge_start[:-1].contiguous(), lens.to(torch.int32).contiguous()
        fn = _lib.bind("rb200_ctc_fsa", [_vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp])
        _lib.check(fn(tg.data_ptr(), tg.shape[1] if tg.dim() > 1 else 0, l32.data_ptr(), sb32.data_ptr(), eb32.data_ptr(), B, int(blank),
                      1 if label_loop else 0, e_from.data_ptr(), e_to.data_ptr(), e_em.data_ptr(), w.data_ptr(), start.data_ptr(), end.data_ptr(),
                      end2.data_ptr(), _lib.stream_ptr()), "ctc_fsa")
        _lib.count_launch()
        return FsaBatch(e_from, e_to, e_em, w, edge_start, start, end, end2, S_total)
    # host construction (same slot layout)
    tg_l, lens_l, base_l = tg.cpu().tolist(), lens.cpu().tolist(), state_base.cpu().tolist()
    ef, et, ee, ww, st, en, en2 = [], [], [], [], [], [], []
    inf = float("inf")
    for b in range(B):
        Sb, sb = lens_l[b], base_l[b]
        n = 2 * Sb + 1
        sym = lambda s: tg_l[b][s // 2] if s & 1 else blank  # noqa: E731
        st.append(sb); en.append(sb + n - 1); en2.append(sb + n - 2 if Sb > 0 else -1)
        for s in range(n):
            is_label = bool(s & 1)
            ef.append(sb + s); et.append(sb + s); ee.append(sym(s)); ww.append(0.0 if (not is_label or label_loop) else inf)
            if s + 1 < n:
                ef.append(sb + s); et.append(sb + s + 1); ee.append(sym(s + 1)); ww.append(0.0)
            else:
                ef.append(sb); et.append(sb); ee.append(blank); ww.append(inf)
            if is_label and s + 2 < n and sym(s) != sym(s + 2):
                ef.append(sb + s); et.append(sb + s + 2); ee.append(sym(s + 2)); ww.append(0.0)
            else:
                ef.append(sb); et.append(sb); ee.append(blank); ww.append(inf)
    mk = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt, device=dev)  # noqa: E731
    return FsaBatch(mk(ef), mk(et), mk(ee), mk(ww, torch.float32), edge_start, mk(st), mk(en), mk(en2), S_total)


def _scatter_logsumexp(scores: torch.Tensor, index: torch.Tensor, size: int) -> torch.Tensor:
    m = torch.full((size,), float("-inf"), dtype=scores.dtype, device=scores.device).scatter_reduce(0, index, scores, reduce="amax", include_self=True)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    s = torch.zeros(size, dtype=scores.dtype, device=scores.device).scatter_add(0, index, torch.exp(scores - m_safe[index]))
    return torch.where(s > 0, m_safe + torch.log(s), torch.full_like(m, float("-inf")))


def fast_baum_welch_reference(am_scores: torch.Tensor, fsa: FsaBatch, lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch implementation, one frame per iteration, vectorised over all edges of the batch"""
    T, B, V = am_scores.shape
    dev = am_scores.device
    S = fsa.num_states
    seq = fsa.edge_seq()
    ef, et, ee = fsa.e_from.long(), fsa.e_to.long(), fsa.e_em.long()
    lens_d = lens.to(dev)
    ninf = float("-inf")
    fwd = [torch.full((S,), ninf, device=dev).index_fill(0, fsa.start.long(), 0.0)]
    for t in range(T):
        active = (t < lens_d)[seq]
        sc = fwd[t][ef] - fsa.weights - am_scores[t, seq, ee]
        sc = torch.where(active, sc, torch.full_like(sc, ninf))
        fwd.append(_scatter_logsumexp(sc, et, S))
    # backward starts at each sequence's own length
    bwd_t = torch.full((T + 1, S), ninf, device=dev)
    for b in range(B):
        Tb = int(lens[b])
        bwd_t[Tb, int(fsa.end[b])] = 0.0
        if int(fsa.end2[b]) >= 0:
            bwd_t[Tb, int(fsa.end2[b])] = 0.0
    for t in range(T - 1, -1, -1):
        active = (t < lens_d)[seq]
        sc = bwd_t[t + 1][et] - fsa.weights - am_scores[t, seq, ee]
        sc = torch.where(active, sc, torch.full_like(sc, ninf))
        cur = _scatter_logsumexp(sc, ef, S)
        # a sequence that ends at t has its final states initialised in row t: merge
        bwd_t[t] = torch.where(torch.isinf(bwd_t[t]), cur, torch.logaddexp(bwd_t[t], cur))
    total = bwd_t[0][fsa.start.long()]  # [B]
    out = torch.full((T, B, V), ninf, device=dev)
    for t in range(T):
        active = (t < lens_d)[seq]
        sc = fwd[t][ef] - fsa.weights - am_scores[t, seq, ee] + bwd_t[t + 1][et] - total[seq]
        sc = torch.where(active, sc, torch.full_like(sc, ninf))
        flat = _scatter_logsumexp(sc, seq * V + ee, B * V)
        out[t] = flat.reshape(B, V)
    return -out, -total


def fast_baum_welch(am_scores: torch.Tensor, fsa: FsaBatch, lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    :param am_scores: [T, B, V] negative log scores per frame and emission label
    :param lens: [B] number of frames per sequence
    :return: (fwdbwd [T, B, V] = -log posterior of the label at that frame (+inf where impossible), obs_scores [B] = -log total score)
    """
    T, B, V = am_scores.shape
    if _native(am_scores, "rb200_fsa_fbw"):
        dev = am_scores.device
        am = am_scores.float().contiguous()
        S = fsa.num_states
        fwd = torch.full((T + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        bwd = torch.full((T + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        out = torch.full((T, B, V), float("-inf"), dtype=torch.float32, device=dev)
        obs = torch.empty(B, dtype=torch.float32, device=dev)
        l32 = lens.to(dev, torch.int32).contiguous()
        fn = _lib.bind("rb200_fsa_fbw", [_vp] * 10 + [_i32] * 4 + [_vp] * 5)
        _lib.check(fn(fsa.e_from.data_ptr(), fsa.e_to.data_ptr(), fsa.e_em.data_ptr(), fsa.weights.data_ptr(), fsa.edge_start.data_ptr(), am.data_ptr(),
                      fsa.start.data_ptr(), fsa.end.data_ptr(), fsa.end2.data_ptr(), l32.data_ptr(), T, B, V, S, fwd.data_ptr(), bwd.data_ptr(),
                      out.data_ptr(), obs.data_ptr(), _lib.stream_ptr()), "fsa_fbw")
        _lib.count_launch()
        return -out, -obs
    return fast_baum_welch_reference(am_scores.float(), fsa, lens)


def fast_baum_welch_packed(am_scores: torch.Tensor, fsa: FsaBatch, *, row_start: torch.Tensor, lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    :func:`fast_baum_welch` on packed scores (FastBaumWelchPackedOp, returnn/native_op.py:3754).

    :param am_scores: [N, V] negative log scores, the frames of sequence b are rows ``row_start[b] .. row_start[b] + lens[b]``
    :return: (fwdbwd [N, V] -log posteriors, obs_scores [B])
    """
    N, V = am_scores.shape
    B = fsa.batch
    dev = am_scores.device
    t_max = int(lens.max()) if B else 0
    if _native(am_scores, "rb200_fsa_fbw_packed"):
        am = am_scores.float().contiguous()
        S = fsa.num_states
        fwd = torch.full((t_max + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        bwd = torch.full((t_max + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        out = torch.full((N, V), float("-inf"), dtype=torch.float32, device=dev)
        obs = torch.empty(B, dtype=torch.float32, device=dev)
        l32 = lens.to(dev, torch.int32).contiguous()
        rs = row_start.to(dev, torch.int32).contiguous()
        fn = _lib.bind("rb200_fsa_fbw_packed", [_vp] * 11 + [_i32] * 4 + [_vp] * 5)
        _lib.check(fn(fsa.e_from.data_ptr(), fsa.e_to.data_ptr(), fsa.e_em.data_ptr(), fsa.weights.data_ptr(), fsa.edge_start.data_ptr(), am.data_ptr(),
                      fsa.start.data_ptr(), fsa.end.data_ptr(), fsa.end2.data_ptr(), l32.data_ptr(), rs.data_ptr(), t_max, B, V, S, fwd.data_ptr(),
                      bwd.data_ptr(), out.data_ptr(), obs.data_ptr(), _lib.stream_ptr()), "fsa_fbw_packed")
        _lib.count_launch()
        return -out, -obs
    padded = torch.zeros(t_max, B, V, dtype=torch.float32, device=dev)
    for b in range(B):
        padded[: int(lens[b]), b] = am_scores[int(row_start[b]): int(row_start[b]) + int(lens[b])].float()
    res, obs = fast_baum_welch(padded, fsa, lens)
    out = torch.full((N, V), float("inf"), dtype=torch.float32, device=dev)
    for b in range(B):
        out[int(row_start[b]): int(row_start[b]) + int(lens[b])] = res[: int(lens[b]), b]
    return out, obs


def fast_baum_welch_multi_end_reference(am_scores: torch.Tensor, fsa: FsaBatch, lens: torch.Tensor, end_start: torch.Tensor, end_state: torch.Tensor,
                                        end_weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch implementation of :func:`fast_baum_welch_multi_end`"""
    T, B, V = am_scores.shape
    dev = am_scores.device
    S = fsa.num_states
    seq = fsa.edge_seq()
    ef, et, ee = fsa.e_from.long(), fsa.e_to.long(), fsa.e_em.long()
    lens_d = lens.to(dev)
    ninf = float("-inf")
    fwd = [torch.full((S,), ninf, device=dev).index_fill(0, fsa.start.long(), 0.0)]
    for t in range(T):
        active = (t < lens_d)[seq]
        sc = torch.where(active, fwd[t][ef] - fsa.weights - am_scores[t, seq, ee], torch.full((ef.shape[0],), ninf, device=dev))
        fwd.append(_scatter_logsumexp(sc, et, S))
    bwd_t = torch.full((T + 1, S), ninf, device=dev)
    es = end_start.tolist()
    for b in range(B):
        Tb = int(lens[b])
        for i in range(es[b], es[b + 1]):
            st = int(end_state[i])
            bwd_t[Tb, st] = torch.logaddexp(bwd_t[Tb, st], -end_weight[i].to(dev))
    for t in range(T - 1, -1, -1):
        active = (t < lens_d)[seq]
        sc = torch.where(active, bwd_t[t + 1][et] - fsa.weights - am_scores[t, seq, ee], torch.full((ef.shape[0],), ninf, device=dev))
        cur = _scatter_logsumexp(sc, ef, S)
        bwd_t[t] = torch.where(torch.isinf(bwd_t[t]), cur, torch.logaddexp(bwd_t[t], cur))
    total = bwd_t[0][fsa.start.long()]
    out = torch.full((T, B, V), ninf, device=dev)
    for t in range(T):
        active = (t < lens_d)[seq]
        sc = fwd[t][ef] - fsa.weights - am_scores[t, seq, ee] + bwd_t[t + 1][et] - total[seq]
        sc = torch.where(active, sc, torch.full_like(sc, ninf))
        out[t] = _scatter_logsumexp(sc, seq * V + ee, B * V).reshape(B, V)
    return -out, -total


def fast_baum_welch_multi_end(am_scores: torch.Tensor, fsa: FsaBatch, lens: torch.Tensor, *, end_states: torch.Tensor,
                              end_state_weights: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    Full-sum forward-backward where every sequence may end in several states, each with its own weight
    (``fsa.end`` / ``fsa.end2`` are not used).

    :param am_scores: [T, B, V] negative log scores
    :param end_states: [N, 2] int: (sequence index, state index), in any order
    :param end_state_weights: [N] negative log weight of ending in that state
    :return: (fwdbwd [T, B, V] -log posteriors, obs_scores [B] -log total score incl. the end weights)
    """
    T, B, V = am_scores.shape
    dev = am_scores.device
    es = end_states.to(dev).long()
    order = torch.argsort(es[:, 0], stable=True)
    seq_of = es[order, 0]
    end_state = es[order, 1].to(torch.int32).contiguous()
    end_weight = end_state_weights.to(dev, torch.float32)[order].contiguous()
    counts = torch.bincount(seq_of, minlength=B)
    end_start = torch.zeros(B + 1, dtype=torch.int32, device=dev)
    end_start[1:] = torch.cumsum(counts, 0).to(torch.int32)
    if _native(am_scores, "rb200_fsa_fbw_multi_end"):
        am = am_scores.float().contiguous()
        S = fsa.num_states
        fwd = torch.full((T + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        bwd = torch.full((T + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        out = torch.full((T, B, V), float("-inf"), dtype=torch.float32, device=dev)
        obs = torch.empty(B, dtype=torch.float32, device=dev)
        l32 = lens.to(dev, torch.int32).contiguous()
        fn = _lib.bind("rb200_fsa_fbw_multi_end", [_vp] * 11 + [_i32] * 4 + [_vp] * 5)
        _lib.check(fn(fsa.e_from.data_ptr(), fsa.e_to.data_ptr(), fsa.e_em.data_ptr(), fsa.weights.data_ptr(), fsa.edge_start.data_ptr(), am.data_ptr(),
                      fsa.start.data_ptr(), end_start.data_ptr(), end_state.data_ptr(), end_weight.data_ptr(), l32.data_ptr(), T, B, V, S,
                      fwd.data_ptr(), bwd.data_ptr(), out.data_ptr(), obs.data_ptr(), _lib.stream_ptr()), "fsa_fbw_multi_end")
        _lib.count_launch()
        return -out, -obs
    return fast_baum_welch_multi_end_reference(am_scores.float(), fsa, lens, end_start.cpu(), end_state, end_weight)


def segment_fast_baum_welch_reference(am_scores: torch.Tensor, fsa: FsaBatch, e_lenmod: torch.Tensor, length_models: torch.Tensor, row_start: torch.Tensor,
                                      lens: torch.Tensor, am_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch implementation of :func:`segment_fast_baum_welch`: a loop over frames, vectorised over (edge, length)"""
    N, L, V = am_scores.shape
    dev = am_scores.device
    S = fsa.num_states
    B = fsa.batch
    seq = fsa.edge_seq()
    ef, et, ee, lm = fsa.e_from.long(), fsa.e_to.long(), fsa.e_em.long(), e_lenmod.long().to(dev)
    lens_d = lens.to(dev).long()
    rows = row_start.to(dev).long()
    T = int(lens.max()) if B else 0
    ninf = float("-inf")
    E = ef.shape[0]
    ar = torch.arange(L, device=dev)

    def costs(t: int):
        """[E, L] cost of every edge with every length at start frame t; +inf where the segment leaves the sequence"""
        row = torch.clamp(rows[seq] + t, max=N - 1)
        c = fsa.weights[:, None] + am_scale * am_scores[row[:, None], ar[None, :], ee[:, None]] + length_models.to(dev)[lm]
        ok = (t + ar[None, :] + 1) <= lens_d[seq][:, None]
        return torch.where(ok, c, torch.full_like(c, float("inf")))

    fwd = torch.full((T + L + 1, S), ninf, device=dev)
    fwd[0, fsa.start.long()] = 0.0
    for t in range(T):
        sc = fwd[t][ef][:, None] - costs(t)  # [E, L]
        for l in range(L):
            upd = _scatter_logsumexp(sc[:, l], et, S)
            fwd[t + l + 1] = torch.logaddexp(fwd[t + l + 1], upd)
    bwd = torch.full((T + L + 1, S), ninf, device=dev)
    for b in range(B):
        bwd[int(lens[b]), int(fsa.end[b])] = 0.0
    for t in range(T - 1, -1, -1):
        c = costs(t)
        nxt = torch.stack([bwd[t + l + 1][et] for l in range(L)], dim=1)  # [E, L]
        sc = torch.logsumexp(nxt - c, dim=1)
        cur = _scatter_logsumexp(sc, ef, S)
        bwd[t] = torch.logaddexp(bwd[t], cur)
    total = bwd[0][fsa.start.long()]
    out = torch.full((N * L * V,), ninf, device=dev)
    for t in range(T):
        c = costs(t)
        nxt = torch.stack([bwd[t + l + 1][et] for l in range(L)], dim=1)
        sc = fwd[t][ef][:, None] - c + nxt - total[seq][:, None]  # [E, L]
        row = torch.clamp(rows[seq] + t, max=N - 1)
        idx = (row[:, None] * L + ar[None, :]) * V + ee[:, None]
        valid = torch.isfinite(sc)
        upd = _scatter_logsumexp(torch.where(valid, sc, torch.full_like(sc, ninf)).reshape(-1), idx.reshape(-1), N * L * V)
        out = torch.logaddexp(out, upd)
    return -out.reshape(N, L, V), -total


def segment_fast_baum_welch(am_scores: torch.Tensor, fsa: FsaBatch, *, e_lenmod: torch.Tensor, length_models: torch.Tensor, row_start: torch.Tensor,
                            lens: torch.Tensor, am_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    Segmental full-sum: an edge taken at frame ``t`` consumes ``l`` = 1 .. L frames and costs
    ``weight + am_scale * am_scores[row_start[b] + t, l - 1, emission] + length_models[e_lenmod[e], l - 1]``.

    :param am_scores: [N, L, V] negative log scores, one row per (sequence, segment start frame); the rows of sequence b are
        ``row_start[b] .. row_start[b] + lens[b]``
    :param e_lenmod: [E] int: which length model each edge uses
    :param length_models: [M, L] negative log probability of every segment length
    :return: (posteriors [N, L, V] as -log of P(a segment with this start, length and label), obs_scores [B])
    """
    N, L, V = am_scores.shape
    dev = am_scores.device
    if _native(am_scores, "rb200_fsa_seg_fbw"):
        am = am_scores.float().contiguous()
        S, B = fsa.num_states, fsa.batch
        t_max = int(lens.max()) if B else 0
        fwd = torch.full((t_max + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        bwd = torch.full((t_max + 1, S), float("-inf"), dtype=torch.float32, device=dev)
        out = torch.full((N, L, V), float("-inf"), dtype=torch.float32, device=dev)
        obs = torch.empty(B, dtype=torch.float32, device=dev)
        l32 = lens.to(dev, torch.int32).contiguous()
        rs = row_start.to(dev, torch.int32).contiguous()
        lm = e_lenmod.to(dev, torch.int32).contiguous()
        lmod = length_models.to(dev, torch.float32).contiguous()
        fn = _lib.bind("rb200_fsa_seg_fbw", [_vp] * 12 + [_i32] * 5 + [ctypes.c_float] + [_vp] * 5)
        _lib.check(fn(fsa.e_from.data_ptr(), fsa.e_to.data_ptr(), fsa.e_em.data_ptr(), lm.data_ptr(), fsa.weights.data_ptr(), fsa.edge_start.data_ptr(),
                      am.data_ptr(), lmod.data_ptr(), rs.data_ptr(), fsa.start.data_ptr(), fsa.end.data_ptr(), l32.data_ptr(), B, L, V, S, t_max,
                      float(am_scale), fwd.data_ptr(), bwd.data_ptr(), out.data_ptr(), obs.data_ptr(), _lib.stream_ptr()), "fsa_seg_fbw")
        _lib.count_launch()
        return -out, -obs
    return segment_fast_baum_welch_reference(am_scores.float(), fsa, e_lenmod, length_models.float(), row_start, lens, am_scale)


def fast_viterbi_reference(am_scores: torch.Tensor, fsa: FsaBatch, lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """host loop (small inputs)"""
    T, B, V = am_scores.shape
    am = am_scores.float().cpu()
    ef, et, ee, w = fsa.e_from.cpu().tolist(), fsa.e_to.cpu().tolist(), fsa.e_em.cpu().tolist(), fsa.weights.cpu().tolist()
    es = fsa.edge_start.cpu().tolist()
    align = torch.zeros(T, B, dtype=torch.int32)
    best = torch.full((B,), float("-inf"))
    for b in range(B):
        Tb = int(lens[b])
        score = {int(fsa.start[b]): 0.0}
        back = []
        for t in range(Tb):
            nxt, bp = {}, {}
            for e in range(es[b], es[b + 1]):
                if ef[e] in score and w[e] != float("inf"):
                    s = score[ef[e]] - w[e] - float(am[t, b, ee[e]])
                    if et[e] not in nxt or s > nxt[et[e]]:
                        nxt[et[e]], bp[et[e]] = s, e
            score = nxt
            back.append(bp)
        cands = [(score[s], s) for s in (int(fsa.end[b]), int(fsa.end2[b])) if s in score]
        if not cands:
            continue
        sc, st = max(cands)
        best[b] = sc
        for t in range(Tb - 1, -1, -1):
            e = back[t][st]
            align[t, b] = ee[e]
            st = ef[e]
    return align.to(am_scores.device), (-best).to(am_scores.device)


def fast_viterbi(am_scores: torch.Tensor, fsa: FsaBatch, lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    :return: (alignment [T, B] int32 = emission label of the best path per frame (0 after the end), scores [B] = -log score of the best path)
    """
    T, B, V = am_scores.shape
    if _native(am_scores, "rb200_fsa_viterbi"):
        dev = am_scores.device
        am = am_scores.float().contiguous()
        S = fsa.num_states
        score = torch.zeros((T + 1) * S, dtype=torch.int64, device=dev)
        align = torch.empty(T, B, dtype=torch.int32, device=dev)
        best = torch.empty(B, dtype=torch.float32, device=dev)
        l32 = lens.to(dev, torch.int32).contiguous()
        fn = _lib.bind("rb200_fsa_viterbi", [_vp] * 10 + [_i32] * 4 + [_vp] * 4)
        _lib.check(fn(fsa.e_from.data_ptr(), fsa.e_to.data_ptr(), fsa.e_em.data_ptr(), fsa.weights.data_ptr(), fsa.edge_start.data_ptr(), am.data_ptr(),
                      fsa.start.data_ptr(), fsa.end.data_ptr(), fsa.end2.data_ptr(), l32.data_ptr(), T, B, V, S, score.data_ptr(), align.data_ptr(),
                      best.data_ptr(), _lib.stream_ptr()), "fsa_viterbi")
        _lib.count_launch()
        return align, -best
    return fast_viterbi_reference(am_scores, fsa, lens)


class _CtcViaFsaFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_tbv, fsa, lens):
        log_probs = torch.log_softmax(logits_tbv.float(), dim=-1)
        fwdbwd, obs = fast_baum_welch(-log_probs, fsa, lens)
        T = logits_tbv.shape[0]
        mask = (torch.arange(T, device=logits_tbv.device)[:, None] < lens.to(logits_tbv.device)[None, :]).unsqueeze(-1)
        # d loss / d logits = softmax - posterior (inside the sequence)
        grad = (torch.exp(log_probs) - torch.exp(-fwdbwd)) * mask
        feasible = torch.isfinite(obs)
        ctx.save_for_backward(grad * feasible[None, :, None])
        ctx.dtype = logits_tbv.dtype
        return torch.where(feasible, obs, torch.zeros_like(obs))

    @staticmethod
    def backward(ctx, dloss):
        (grad,) = ctx.saved_tensors
        return (grad * dloss.float()[None, :, None]).to(ctx.dtype), None, None


def ctc_loss_via_fsa(logits: torch.Tensor, targets: torch.Tensor, in_lens: torch.Tensor, tgt_lens: torch.Tensor, *, blank: int,
                     label_loop: bool = True) -> torch.Tensor:
    """
    CTC loss computed as a full sum over the CTC FSA (the generic route, which also serves other topologies).

    :param logits: [B, T, V] unnormalised
    :return: [B] loss (0 where no alignment exists)
    """
    fsa = ctc_fsa(targets, tgt_lens, blank=blank, label_loop=label_loop)
    return _CtcViaFsaFn.apply(logits.transpose(0, 1), fsa, in_lens)
