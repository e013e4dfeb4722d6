"""
Sequence utility ops with B200 kernels (``csrc/seq_ops.cu``) and plain torch / numpy references that also serve as the CPU path:

- :func:`device_assert`: asynchronous check of a device condition; a failure is recorded in a status word that
  :func:`check_asserts` reads later (no trap, the context stays usable)
- :func:`edit_distance` (reference: returnn/native_op.py:5866 EditDistanceOp)
- :func:`beam_topk`: one beam-search step (log-softmax + accumulated scores + top-k over beam x vocab + backrefs)
- :func:`rnnt_loss`: transducer loss on gathered blank / label log-probabilities
"""

from __future__ import annotations
from typing import Dict, List, Optional, Tuple
import ctypes
import torch
from . import _lib

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_assert_status: Dict[str, torch.Tensor] = {}
_assert_messages: Dict[int, str] = {}


def _native(t: torch.Tensor, name: str) -> bool:
    return t.is_cuda and _lib.use_native(t) and hasattr(_lib.get_lib(), name)


def device_assert(cond: torch.Tensor, message: str = "device assert failed"):
    """
    Check that all elements of ``cond`` (bool) are true without synchronising. On CUDA the check runs as a kernel that records
    the failure; call :func:`check_asserts` (e.g. once per step) to raise. On CPU it raises immediately.
    """
    if not cond.is_cuda:
        if not bool(cond.all()):
            raise AssertionError(message)
        return
    code = len(_assert_messages) + 1
    _assert_messages[code] = message
    key = str(cond.device)
    st = _assert_status.get(key)
    if st is None:
        st = torch.zeros(2, dtype=torch.int32, device=cond.device)
        _assert_status[key] = st
    c = cond.to(torch.uint8).contiguous()
    if _native(c, "rb200_device_assert"):
        fn = _lib.bind("rb200_device_assert", [_vp, _i64, _vp, _i32, _vp])
        _lib.check(fn(c.data_ptr(), c.numel(), st.data_ptr(), code, _lib.stream_ptr()), "device_assert")
        _lib.count_launch()
    else:
        bad = (c == 0).reshape(-1)
        st[0] = torch.where(bad.any() & (st[0] == 0), torch.tensor(code, device=c.device, dtype=torch.int32), st[0])


def check_asserts():
    """raise AssertionError for the first recorded failure (synchronises)"""
    for key, st in _assert_status.items():
        code, idx = [int(v) for v in st.tolist()]
        if code:
            st.zero_()
            raise AssertionError("%s (first failing element %i, device %s)" % (_assert_messages.get(code, "device assert failed"), idx, key))


def edit_distance_reference(a: torch.Tensor, a_len: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor) -> torch.Tensor:
    """Levenshtein distance per row, on the host"""
    out = []
    a_, b_ = a.cpu().tolist(), b.cpu().tolist()
    for i, (n, m) in enumerate(zip(a_len.cpu().tolist(), b_len.cpu().tolist())):
        x, y = a_[i][:n], b_[i][:m]
        prev = list(range(m + 1))
        for p in range(1, n + 1):
            cur = [p] + [0] * m
            for q in range(1, m + 1):
                cur[q] = min(prev[q] + 1, cur[q - 1] + 1, prev[q - 1] + (x[p - 1] != y[q - 1]))
            prev = cur
        out.append(prev[m])
    return torch.tensor(out, dtype=torch.int32, device=a.device)


def edit_distance(a: torch.Tensor, a_len: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor) -> torch.Tensor:
    """
    :param a: [B, La] int labels (padded), ``a_len`` [B]; likewise b
    :return: [B] int32 number of substitutions + insertions + deletions
    """
    if _native(a, "rb200_edit_distance") and b.shape[1] <= 2048:
        a32, b32 = a.to(torch.int32).contiguous(), b.to(torch.int32).contiguous()
        al, bl = a_len.to(a.device, torch.int32).contiguous(), b_len.to(a.device, torch.int32).contiguous()
        out = torch.empty(a.shape[0], dtype=torch.int32, device=a.device)
        fn = _lib.bind("rb200_edit_distance", [_vp, _vp, _i32, _vp, _vp, _i32, _vp, _i32, _i32, _vp])
        _lib.check(fn(a32.data_ptr(), al.data_ptr(), a32.shape[1], b32.data_ptr(), bl.data_ptr(), b32.shape[1], out.data_ptr(), a.shape[0],
                      b32.shape[1], _lib.stream_ptr()), "edit_distance")
        _lib.count_launch()
        return out
    return edit_distance_reference(a, a_len, b, b_len)


def beam_topk_reference(logits, prev_scores, finished, eos: int, k: int, normalized: bool = False):
    """plain torch"""
    B, beam, V = logits.shape
    lp = logits.float() if normalized else torch.log_softmax(logits.float(), dim=-1)
    scores = prev_scores[:, :, None] + lp
    if finished is not None:
        fin = finished.bool()[:, :, None]
        only_eos = torch.full_like(scores, float("-inf"))
        only_eos[:, :, eos] = prev_scores
        scores = torch.where(fin, only_eos, scores)
    top, idx = torch.topk(scores.reshape(B, beam * V), k, dim=-1)
    return top, (idx // V).to(torch.int32), (idx % V).to(torch.int32)


def beam_topk(logits: torch.Tensor, prev_scores: torch.Tensor, *, finished: Optional[torch.Tensor] = None, eos: int = 0, k: int,
              normalized: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    :param logits: [B, beam, V] scores of the next label (fp32 / bf16); log-softmax is applied unless ``normalized``
    :param prev_scores: [B, beam] accumulated log scores
    :param finished: [B, beam] bool: finished hypotheses keep their score and only continue with ``eos``
    :return: (scores [B, k], backrefs [B, k] int32 = source beam index, labels [B, k] int32), sorted by score
    """
    B, beam, V = logits.shape
    if _native(logits, "rb200_beam_topk") and k <= 32 and beam <= 64 and logits.dtype in (torch.float32, torch.bfloat16):
        lg = logits.contiguous()
        ps = prev_scores.float().contiguous()
        fin = finished.to(torch.uint8).contiguous() if finished is not None else None
        dev = logits.device
        out_s = torch.empty(B, k, dtype=torch.float32, device=dev)
        out_b = torch.empty(B, k, dtype=torch.int32, device=dev)
        out_l = torch.empty(B, k, dtype=torch.int32, device=dev)
        kt = 8 if k <= 8 else (16 if k <= 16 else 32)
        scratch = torch.empty(B * beam * kt * 2, dtype=torch.int32, device=dev)  # (score, index) per candidate of the per-row stage
        fn = _lib.bind("rb200_beam_topk", [_vp, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp])
        _lib.check(fn(lg.data_ptr(), 1 if lg.dtype == torch.bfloat16 else 0, 1 if normalized else 0, ps.data_ptr(),
                      fin.data_ptr() if fin is not None else None, B, beam, V, int(eos), int(k), out_s.data_ptr(), out_b.data_ptr(), out_l.data_ptr(),
                      scratch.data_ptr(), _lib.stream_ptr()), "beam_topk")
        _lib.count_launch(2)
        return out_s, out_b, out_l
    return beam_topk_reference(logits, prev_scores, finished, eos, k, normalized)


def rnnt_loss_reference(lp_blank: torch.Tensor, lp_label: torch.Tensor, t_lens: torch.Tensor, u_lens: torch.Tensor) -> torch.Tensor:
    """differentiable torch implementation of the lattice recursion (loops over anti-diagonals)"""
    B, T, U1 = lp_blank.shape
    losses = []
    for b in range(B):
        Tb, Ub = int(t_lens[b]), int(u_lens[b]) + 1
        alpha = [[None] * Ub for _ in range(Tb)]
        for t in range(Tb):
            for u in range(Ub):
                if t == 0 and u == 0:
                    alpha[t][u] = lp_blank.new_zeros(())
                    continue
                terms = []
                if t > 0:
                    terms.append(alpha[t - 1][u] + lp_blank[b, t - 1, u])
                if u > 0:
                    terms.append(alpha[t][u - 1] + lp_label[b, t, u - 1])
                alpha[t][u] = torch.logsumexp(torch.stack(terms), dim=0)
        losses.append(-(alpha[Tb - 1][Ub - 1] + lp_blank[b, Tb - 1, Ub - 1]) if Tb > 0 else lp_blank.new_zeros(()))
    return torch.stack(losses)


class _RnntFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lp_blank, lp_label, t_lens, u_lens):
        B, T, U1 = lp_blank.shape
        pb, pl = lp_blank.float().contiguous(), lp_label.float().contiguous()
        dev = pb.device
        alpha = torch.empty(B, T, U1, dtype=torch.float32, device=dev)
        beta = torch.empty(B, T, U1, dtype=torch.float32, device=dev)
        loss = torch.empty(B, dtype=torch.float32, device=dev)
        need = lp_blank.requires_grad or lp_label.requires_grad
        db = torch.empty_like(pb) if need else None
        dl = torch.empty_like(pl) if need else None
        fn = _lib.bind("rb200_rnnt_loss", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp])
        _lib.check(fn(pb.data_ptr(), pl.data_ptr(), t_lens.data_ptr(), u_lens.data_ptr(), B, T, U1, alpha.data_ptr(), beta.data_ptr(), loss.data_ptr(),
                      db.data_ptr() if need else None, dl.data_ptr() if need else None, _lib.stream_ptr()), "rnnt_loss")
        _lib.count_launch()
        if need:
            ctx.save_for_backward(db, dl)
        ctx.dtypes = (lp_blank.dtype, lp_label.dtype)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        db, dl = ctx.saved_tensors
        s = dloss.float()[:, None, None]
        return (db * s).to(ctx.dtypes[0]), (dl * s).to(ctx.dtypes[1]), None, None


def rnnt_loss(lp_blank: torch.Tensor, lp_label: torch.Tensor, t_lens: torch.Tensor, u_lens: torch.Tensor) -> torch.Tensor:
    """
    Transducer negative log likelihood.

    :param lp_blank: [B, T, U+1] log-probability of blank at lattice node (t, u)
    :param lp_label: [B, T, U+1] log-probability of the (u+1)-th target label at node (t, u) (last column unused)
    :param t_lens: [B] encoder lengths; u_lens: [B] label lengths
    :return: [B] loss
    """
    if _native(lp_blank, "rb200_rnnt_loss"):
        tl = t_lens.to(lp_blank.device, torch.int32).contiguous()
        ul = u_lens.to(lp_blank.device, torch.int32).contiguous()
        return _RnntFn.apply(lp_blank, lp_label, tl, ul)
    return rnnt_loss_reference(lp_blank, lp_label, t_lens, u_lens)


def rnnt_loss_from_joint(joint_logits: torch.Tensor, targets: torch.Tensor, t_lens: torch.Tensor, u_lens: torch.Tensor, blank: int = 0) -> torch.Tensor:
    """
    :param joint_logits: [B, T, U+1, V] unnormalised joint network output
    :param targets: [B, U] labels
    """
    lp = torch.log_softmax(joint_logits.float(), dim=-1)
    lp_blank = lp[..., blank]
    B, T, U1, V = lp.shape
    tgt = torch.cat([targets.long(), targets.new_zeros(B, 1).long()], dim=1)[:, None, :, None].expand(B, T, U1, 1)
    lp_label = torch.gather(lp, -1, tgt).squeeze(-1)
    return rnnt_loss(lp_blank, lp_label, t_lens, u_lens)
