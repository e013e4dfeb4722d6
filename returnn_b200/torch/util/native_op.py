"""
The native sequence ops under the names of the reference's torch wrapper module (returnn/torch/util/native_op.py): CTC through
Baum-Welch, Viterbi, best path, and the edit-distance family including the row-wise forms used inside decoding loops. The heavy ops
are the in-tree sm_100a kernels of :mod:`returnn_b200.ops` (see :mod:`returnn_b200.native_op` for the table); the row-wise edit-distance
ops are vectorised tensor programs (one cumulative minimum per row instead of a sequential loop per batch entry).

The reference generates and compiles its ops at first use (``OpMaker``); here they are prebuilt, and ``OpMaker`` / ``make_op`` /
``make_fast_baum_welch_op`` exist as thin adapters for code that asks for an op object.
"""

from __future__ import annotations
from typing import Optional, Tuple, Union
import torch

from ... import native_op as _nop
from ...ops import fsa as _fsa
from ...ops import seq_ops as _seq
from ...ops import ctc as _ctc
from ...ops.fsa import FsaBatch

get_ctc_fsa_fast_bw = _nop.get_ctc_fsa_fast_bw
fast_baum_welch = _nop.fast_baum_welch
fast_viterbi = _nop.fast_viterbi
ctc_loss = _nop.ctc_loss
edit_distance = _nop.edit_distance


class OpMaker:
    """adapter: ``OpMaker(description).make_op()`` returns the prebuilt function of that name"""

    _by_class_name = {
        "FastBaumWelchOp": "fast_baum_welch", "FastViterbiOp": "fast_viterbi", "GetCtcFsaFastBwOp": "get_ctc_fsa_fast_bw",
        "EditDistanceOp": "edit_distance", "OptimalCompletionEditDistanceOp": "optimal_completion_edit_distance",
        "OptimalCompletionEditDistancePerSuccessorOp": "optimal_completion_edit_distance_per_successor",
        "NextEditDistanceRowOp": "next_edit_distance_row", "NextEditDistanceReduceOp": "next_edit_distance_reduce"}

    def __init__(self, description, **_kwargs):
        self.description = description
        self.name = getattr(description, "name", None) or getattr(description, "__name__", None) or str(description)

    def make_op(self):
        """the function"""
        fn_name = self._by_class_name.get(self.name, self.name)
        fn = globals().get(fn_name)
        if fn is None:
            raise NotImplementedError("native op %r has no prebuilt counterpart here" % self.name)
        return fn


def make_op(cls, **kwargs):
    """``make_op(op class or name)`` -> function"""
    return OpMaker(cls, **kwargs).make_op()


def make_fast_baum_welch_op(**_kwargs):
    """the Baum-Welch function (the reference compiles it here)"""
    return fast_baum_welch


def make_fast_baum_welch_packed_op(**_kwargs):
    """the packed-rows Baum-Welch function"""
    return fast_baum_welch_packed


def fast_baum_welch_packed(am_scores: torch.Tensor, fsa: FsaBatch, *, row_start: torch.Tensor, lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """as :func:`fast_baum_welch` on packed score rows ``[sum(len), V]``: ``row_start [B]`` first row of each sequence"""
    return _fsa.fast_baum_welch_packed(am_scores, fsa, row_start=row_start, lens=lens)


def ctc_loss_packed(*, logits: torch.Tensor, pack, targets: torch.Tensor, targets_seq_lens: torch.Tensor, blank_index: int = -1) -> torch.Tensor:
    """CTC loss per sequence on packed logit rows (``pack``: ``models.packing.PackInfo`` of the rows)"""
    if blank_index < 0:
        blank_index += logits.shape[-1]
    return _ctc.ctc_loss_packed(logits, pack, targets, targets_seq_lens.cpu(), blank_index=blank_index)


def ctc_best_path(*, logits: torch.Tensor, logits_seq_lens: torch.Tensor, targets: torch.Tensor, targets_seq_lens: torch.Tensor,
                  blank_index: int = -1, label_loop: bool = True) -> torch.Tensor:
    """
    Viterbi alignment of the targets: ``[B, T]`` label (or blank) per frame, frames beyond a sequence's length hold the blank.
    ``logits`` ``[B, T, V]``.
    """
    if blank_index < 0:
        blank_index += logits.shape[-1]
    log_probs = torch.log_softmax(logits.float(), dim=-1)
    fsa = _fsa.ctc_fsa(targets, targets_seq_lens, blank=blank_index, label_loop=label_loop)
    align, _ = _fsa.fast_viterbi(-log_probs.detach().transpose(0, 1).contiguous(), fsa, logits_seq_lens)
    align = align.transpose(0, 1)
    T = logits.shape[1]
    mask = torch.arange(T, device=logits.device)[None, :] < logits_seq_lens.to(logits.device)[:, None]
    return torch.where(mask, align.to(torch.int32), torch.full_like(align, blank_index, dtype=torch.int32))


# ---- edit distances ---------------------------------------------------------------------------------------------------------------------
def _repeat_last(row: torch.Tensor, b_len: torch.Tensor) -> torch.Tensor:
    """entries beyond ``b_len`` take the value at ``b_len``"""
    n = row.shape[1]
    idx = torch.minimum(torch.arange(n, device=row.device)[None, :], b_len.to(row.device).long()[:, None])
    return torch.gather(row, 1, idx)


def next_edit_distance_row(last_row: torch.Tensor, a: torch.Tensor, a_n: Union[torch.Tensor, int], a_ended: torch.Tensor, b: torch.Tensor,
                           b_len: torch.Tensor) -> torch.Tensor:
    """
    One more symbol of ``a`` against all prefixes of ``b``.

    :param last_row: [B, Tb + 1] int32: distances of ``a[:a_n]`` to ``b[:j]``
    :param a: [B] the symbol at position ``a_n``
    :param a_n: position, scalar or [B]
    :param a_ended: [B] truthy where ``a`` has no symbol at this position any more (the row is copied)
    :param b: [B, Tb], ``b_len`` [B]
    :return: [B, Tb + 1] int32; entries beyond ``b_len`` repeat the entry at ``b_len``
    """
    dev = last_row.device
    B, n = last_row.shape
    if not isinstance(a_n, torch.Tensor):
        a_n = torch.tensor(a_n, device=dev)
    a_n = a_n.to(dev).long().expand(B) if a_n.ndim == 0 else a_n.to(dev).long()
    last = last_row.long()
    sub = last[:, :-1] + (a.to(dev)[:, None] != b.to(dev)).long()  # [B, Tb]: diagonal step
    ins = last[:, 1:] + 1
    c = torch.cat([(a_n + 1)[:, None], torch.minimum(sub, ins)], dim=1)  # candidates without the step along the row
    pos = torch.arange(n, device=dev)[None, :]
    new = torch.cummin(c - pos, dim=1).values + pos  # row steps: new[j] = min_k<=j c[k] + (j - k)
    out = torch.where(a_ended.to(dev).bool()[:, None], last, new)
    return _repeat_last(out, b_len).to(torch.int32)


def edit_distance_via_next_edit_distance_row(a: torch.Tensor, a_len: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor, optimal_completion: bool = False,
                                             full_row_output: bool = False) -> torch.Tensor:
    """the distance built row by row (what a decoding loop does with :func:`next_edit_distance_row`); equal to :func:`edit_distance`"""
    B, t1 = a.shape
    t2 = b.shape[1]
    row = torch.arange(t2 + 1, device=a.device, dtype=torch.int32)[None, :].repeat(B, 1)
    row = _repeat_last(row, b_len)
    for i in range(t1):
        row = next_edit_distance_row(row, a[:, i], i, i >= a_len.to(a.device), b, b_len)
    if full_row_output:
        assert not optimal_completion
        return row
    if not optimal_completion:
        return row[:, -1]
    return row.min(dim=1).values


def optimal_completion_edit_distance(a: torch.Tensor, a_len: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor) -> torch.Tensor:
    """min over the prefixes of ``b`` of the distance to ``a``: what the best continuation of the hypothesis ``a`` can still reach"""
    return edit_distance_via_next_edit_distance_row(a, a_len, b, b_len, optimal_completion=True)


def next_edit_distance_reduce(last_row: torch.Tensor, a: torch.Tensor, a_n: Union[torch.Tensor, int], a_ended: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor,
                              optimal_completion: bool = False, a_blank_idx: Optional[Union[int, torch.Tensor]] = None) -> torch.Tensor:
    """
    For every candidate next symbol at once: the (optimal completion) distance after appending it.

    :param a: [B or 1, n_labels] candidate symbols
    :param a_blank_idx: a candidate equal to this index does not extend ``a`` (the row is kept)
    :return: [B, n_labels] int32
    """
    dev = last_row.device
    B, n = last_row.shape
    a = a.to(dev)
    if a.shape[0] == 1 and B > 1:
        a = a.expand(B, -1)
    L = a.shape[1]
    if not isinstance(a_n, torch.Tensor):
        a_n = torch.tensor(a_n, device=dev)
    a_n = a_n.to(dev).long().expand(B) if a_n.ndim == 0 else a_n.to(dev).long()
    ended = a_ended.to(dev).bool()[:, None].expand(B, L)
    if a_blank_idx is not None and int(a_blank_idx) >= 0:
        ended = ended | (a == int(a_blank_idx))
    rows = next_edit_distance_row(last_row.repeat_interleave(L, dim=0), a.reshape(-1), a_n.repeat_interleave(L), ended.reshape(-1),
                                  b.to(dev).repeat_interleave(L, dim=0), b_len.to(dev).repeat_interleave(L))
    res = rows.min(dim=1).values if optimal_completion else rows[:, -1]
    return res.reshape(B, L).to(torch.int32)


def optimal_completion_edit_distance_per_successor_via_next_edit_distance(a, a_len, b, b_len, successors) -> torch.Tensor:
    """:func:`next_edit_distance_reduce` on the final row of ``a``: [B, n_labels]"""
    if isinstance(successors, int):
        successors = torch.arange(successors, device=a.device)[None]
    elif successors.ndim == 1:
        successors = successors[None]
    last_row = edit_distance_via_next_edit_distance_row(a, a_len, b, b_len, full_row_output=True)
    return next_edit_distance_reduce(last_row, a=successors, a_n=torch.tensor(a.shape[1]), a_ended=a_len.to(a.device) != a.shape[1], b=b, b_len=b_len,
                                     optimal_completion=True)


def optimal_completion_edit_distance_per_successor(a, a_len, b, b_len, successors) -> torch.Tensor:
    """
    For every possible next label of the hypothesis ``a`` (all sequences extended at their own end ``a_len``): the optimal completion
    distance of the extended hypothesis. [B, n_labels]
    """
    if isinstance(successors, int):
        successors = torch.arange(successors, device=a.device)
    dev = a.device
    B, t1 = a.shape
    t2 = b.shape[1]
    row = _repeat_last(torch.arange(t2 + 1, device=dev, dtype=torch.int32)[None, :].repeat(B, 1), b_len)
    for i in range(t1):
        row = next_edit_distance_row(row, a[:, i], i, i >= a_len.to(dev), b, b_len)
    return next_edit_distance_reduce(row, a=successors.to(dev)[None], a_n=a_len.to(dev), a_ended=torch.zeros(B, dtype=torch.bool, device=dev), b=b, b_len=b_len,
                                     optimal_completion=True)
