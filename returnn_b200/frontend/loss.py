"""
Losses and sequence metrics: cross entropy, CTC (loss, greedy decode, best path, durations), edit distance.

Parity: returnn/frontend/loss.py (cross_entropy :22, ctc_loss :66, ctc_greedy_decode :145, edit_distance :326);
CTC backend semantics returnn/torch/frontend/_backend.py:775-869.
"""

from __future__ import annotations
from typing import Optional, Tuple, Union
import torch
import torch.nn.functional as F
from ..tensor import Tensor, Dim, batch_dim
from ._utils import wrap, axis_of

__all__ = ["cross_entropy", "softmax_cross_entropy_smoothed_grad", "ctc_loss", "ctc_best_path", "ctc_durations_from_path", "ctc_no_label_loop_blank_durations_from_path",
           "ctc_greedy_decode", "edit_distance", "mse_loss", "binary_cross_entropy"]


def cross_entropy(*, estimated: Tensor, target: Tensor, axis: Dim, estimated_type: str) -> Tensor:
    """
    ``-sum_axis target * log(estimated)``.

    :param estimated: probs, log-probs or logits over axis
    :param target: sparse class indices (sparse_dim == axis) or a dense distribution over axis
    :param estimated_type: "probs", "log-probs" or "logits"
    :return: dims of estimated without axis
    """
    if estimated_type == "logits" and target.sparse_dim is not None:
        ax = axis_of(estimated, axis)
        rest = [d for d in estimated._dims if d != axis]
        logits = estimated.copy_compatible_to_dims_raw(rest + [axis])
        tgt = target.copy_compatible_to_dims_raw(rest)
        shape = list(logits.shape[:-1])
        if list(tgt.shape) != shape:
            tgt = tgt.expand(*shape)
        if logits.is_cuda and logits.dtype == torch.bfloat16:
            from ..ops import softmax_ce as _ce

            if _ce.available():
                loss = _ce.softmax_cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1), 0.0)
                return wrap(loss.reshape(shape), rest)
        loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt.reshape(-1).long(), reduction="none")
        return wrap(loss.reshape(shape).to(logits.dtype if logits.dtype == torch.float64 else torch.float32), rest)
    from .math_ import log_softmax, safe_log
    from .matmul import matmul
    from .array_ import gather

    if estimated_type == "logits":
        log_prob = log_softmax(estimated, axis=axis)
    elif estimated_type == "log-probs":
        log_prob = estimated
    elif estimated_type == "probs":
        log_prob = safe_log(estimated)
    else:
        raise ValueError("cross_entropy: invalid estimated_type %r" % estimated_type)
    if target.sparse_dim is not None:
        return -gather(log_prob, indices=target, axis=axis)
    return -matmul(target, log_prob, reduce=axis)


def softmax_cross_entropy_smoothed_grad(*, logits: Tensor, target: Tensor, axis: Dim, smoothing: float = 0.0,
                                        with_argmax: bool = False) -> Union[Tensor, Tuple[Tensor, Tensor]]:
    """
    The usual teacher-forced training criterion in one pass over the logits::

        log_prob = rf.log_softmax(logits, axis=axis)
        log_prob = rf.label_smoothed_log_prob_gradient(log_prob, smoothing, axis=axis)
        loss = rf.cross_entropy(target=target, estimated=log_prob, estimated_type="log-probs", axis=axis)
        best = rf.reduce_argmax(logits, axis=axis)          # with_argmax

    On the GPU one kernel reads the logits once in forward (online softmax, target logit, arg max) and once in backward (writes
    ``softmax - (1-s) one_hot - s/V``); the [.., V] log-probabilities, their smoothed gradient and the fp32 copies of the composed
    form are never materialised. Elsewhere the composed form runs.

    :param logits: [..., axis]
    :param target: sparse, sparse_dim == axis
    :param smoothing: label smoothing applied to the gradient only (the loss value is the plain negative log likelihood)
    :param with_argmax: also return the arg max over axis (sparse tensor like target)
    :return: loss with the dims of logits without axis (, arg max)
    """
    from ..ops import softmax_ce as _ce

    rest = [d for d in logits._dims if d != axis]
    raw = logits.copy_compatible_to_dims_raw(rest + [axis])
    tgt = target.copy_compatible_to_dims_raw(rest)
    shape = list(raw.shape[:-1])
    if list(tgt.shape) != shape:
        tgt = tgt.expand(*shape)
    res = _ce.softmax_cross_entropy(raw.reshape(-1, raw.shape[-1]), tgt.reshape(-1), float(smoothing), grad_only_smoothing=True,
                                    with_argmax=with_argmax)
    if not with_argmax:
        return wrap(res.reshape(shape), rest)
    loss, best = res
    best_t = Tensor("argmax", dims=rest, dtype=target.dtype, sparse_dim=axis, raw_tensor=best.reshape(shape).to(tgt.dtype))
    return wrap(loss.reshape(shape), rest), best_t


def mse_loss(estimated: Tensor, target: Tensor) -> Tensor:
    """squared error per element"""
    from .math_ import squared_difference

    return squared_difference(estimated, target)


def binary_cross_entropy(*, estimated: Tensor, target: Tensor, estimated_type: str = "logits") -> Tensor:
    """element-wise BCE"""
    dims = estimated._dims
    t = target.copy_compatible_to_dims_raw(dims).to(estimated._raw_tensor.dtype)
    if estimated_type == "logits":
        return wrap(F.binary_cross_entropy_with_logits(estimated._raw_tensor, t, reduction="none"), dims)
    assert estimated_type == "probs"
    return wrap(F.binary_cross_entropy(estimated._raw_tensor, t, reduction="none"), dims)


def ctc_loss(*, logits: Tensor, logits_normalized: bool = False, targets: Tensor, input_spatial_dim: Dim,
             targets_spatial_dim: Dim, blank_index: int, max_approx: bool = False, use_native_op: Optional[bool] = None,
             label_loop: bool = True) -> Tensor:
    """
    CTC negative log likelihood per sequence.

    On B200 with bf16/fp32 logits the fused sm_100a kernel (log-softmax + alpha/beta recursion + gradient in one pass)
    is used; elsewhere the generic FSA engine (``label_loop=False``, ``max_approx``) or ``torch.nn.functional.ctc_loss``.

    :param logits: [B, T, C] in any order
    :param targets: sparse [B, S]
    :return: [B]
    """
    fd = logits.feature_dim
    assert fd is not None
    batch_dims = [d for d in logits._dims if d not in (input_spatial_dim, fd)]
    assert len(batch_dims) == 1, "ctc_loss: exactly one batch dim expected, got %r" % (batch_dims,)
    bd = batch_dims[0]
    lraw = logits.copy_compatible_to_dims_raw([bd, input_spatial_dim, fd])
    traw = targets.copy_compatible_to_dims_raw([bd, targets_spatial_dim])
    in_lens = _lens(input_spatial_dim, lraw.shape[0], lraw.shape[1])
    tgt_lens = _lens(targets_spatial_dim, traw.shape[0], traw.shape[1])
    if max_approx or not label_loop or use_native_op:
        from .. import native_op

        log_probs = lraw.float() if logits_normalized else F.log_softmax(lraw.float(), dim=-1)
        loss = native_op.ctc_loss(logits=log_probs.transpose(0, 1), logits_normalized=True, logits_seq_lens=in_lens,
                                  logits_time_major=True, targets=traw, targets_seq_lens=tgt_lens, blank_index=blank_index,
                                  label_loop=label_loop, max_approx=max_approx)
        return wrap(loss, [bd])
    if lraw.is_cuda:
        from ..ops import ctc as _ctc

        if _ctc.available() and _ctc.supports(lraw, traw):
            # the kernel wrapper packs the valid frames and needs the lengths on the host: hand them over as they are
            loss = _ctc.ctc_loss(lraw, traw, in_lens, tgt_lens, blank_index=blank_index,
                                 logits_normalized=logits_normalized)
            return wrap(loss, [bd])
    log_probs = lraw.float() if logits_normalized else F.log_softmax(lraw.float(), dim=-1)
    loss = F.ctc_loss(log_probs.transpose(0, 1), traw.long(), in_lens.long().cpu(), tgt_lens.long().cpu(), blank=blank_index,
                      reduction="none", zero_infinity=True)
    return wrap(loss, [bd])


def _lens(dim: Dim, batch: int, max_len: int) -> torch.Tensor:
    if dim.is_dynamic() and dim.dyn_size_ext is not None and dim.dyn_size_ext.dims:
        return dim.dyn_size_ext.raw_tensor.to(torch.int32)
    return torch.full([batch], max_len, dtype=torch.int32)


def ctc_best_path(*, logits: Tensor, logits_normalized: bool = False, targets: Tensor, input_spatial_dim: Dim,
                  targets_spatial_dim: Dim, blank_index: int, label_loop: bool = True) -> Tensor:
    """Viterbi alignment of targets to frames: [B, T] sparse over the classes"""
    from .. import native_op

    fd = logits.feature_dim
    bd = [d for d in logits._dims if d not in (input_spatial_dim, fd)][0]
    lraw = logits.copy_compatible_to_dims_raw([input_spatial_dim, bd, fd]).float()
    if not logits_normalized:
        lraw = F.log_softmax(lraw, dim=-1)
    traw = targets.copy_compatible_to_dims_raw([bd, targets_spatial_dim])
    in_lens = _lens(input_spatial_dim, lraw.shape[1], lraw.shape[0])
    tgt_lens = _lens(targets_spatial_dim, traw.shape[0], traw.shape[1])
    align, _ = native_op.ctc_best_path(log_probs=lraw, seq_lens=in_lens, targets=traw, targets_seq_lens=tgt_lens,
                                       blank_index=blank_index, label_loop=label_loop)
    return wrap(align.to(torch.int32), [input_spatial_dim, bd], sparse_dim=fd).copy_transpose_to_dims([bd, input_spatial_dim])


def ctc_durations_from_path(*, path: Tensor, path_spatial_dim: Dim, blank_index: int,
                            targets_spatial_dim: Optional[Dim] = None, out_spatial_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    Durations of the alternating blank/label state sequence ``[b0, l1, b1, l2, ..., lS, bS]`` of an alignment path:
    [B, 2S+1].
    """
    bd = [d for d in path._dims if d != path_spatial_dim]
    assert len(bd) == 1
    praw = path.copy_compatible_to_dims_raw([bd[0], path_spatial_dim]).cpu()
    lens = _lens(path_spatial_dim, praw.shape[0], praw.shape[1])
    out = []
    for b in range(praw.shape[0]):
        durs = [0]
        prev = blank_index
        for t in range(int(lens[b])):
            c = int(praw[b, t])
            if c == blank_index:
                if len(durs) % 2 == 0:
                    durs.append(0)
                durs[-1] += 1
            else:
                if len(durs) % 2 == 1:
                    durs.append(0)
                elif c != prev:
                    durs.append(0)  # empty blank between two different labels
                    durs.append(0)
                durs[-1] += 1
            prev = c
        if len(durs) % 2 == 0:
            durs.append(0)
        out.append(durs)
    n = max(len(d) for d in out)
    res = torch.zeros(len(out), n, dtype=torch.int32)
    for b, d in enumerate(out):
        res[b, : len(d)] = torch.tensor(d, dtype=torch.int32)
    if out_spatial_dim is None:
        out_spatial_dim = (targets_spatial_dim * 2 + 1) if targets_spatial_dim is not None else Dim(None, name="ctc-durations")
    if out_spatial_dim.is_dynamic() and out_spatial_dim.derived_from_op is None:
        out_spatial_dim.dyn_size_ext = Tensor("durs:size", dims=[bd[0]], dtype="int32", raw_tensor=torch.tensor([len(d) for d in out], dtype=torch.int32))
    return wrap(res.to(path._raw_tensor.device), [bd[0], out_spatial_dim]), out_spatial_dim


def ctc_no_label_loop_blank_durations_from_path(*, path: Tensor, path_spatial_dim: Dim, blank_index: int,
                                                targets_spatial_dim: Optional[Dim] = None, out_spatial_dim: Optional[Dim] = None):
    """blank durations ``[b0, b1, ..., bS]`` for the topology without label loops (each label emitted once)"""
    bd = [d for d in path._dims if d != path_spatial_dim]
    praw = path.copy_compatible_to_dims_raw([bd[0], path_spatial_dim]).cpu()
    lens = _lens(path_spatial_dim, praw.shape[0], praw.shape[1])
    out = []
    for b in range(praw.shape[0]):
        durs = [0]
        for t in range(int(lens[b])):
            if int(praw[b, t]) == blank_index:
                durs[-1] += 1
            else:
                durs.append(0)
        out.append(durs)
    n = max(len(d) for d in out)
    res = torch.zeros(len(out), n, dtype=torch.int32)
    for b, d in enumerate(out):
        res[b, : len(d)] = torch.tensor(d, dtype=torch.int32)
    if out_spatial_dim is None:
        out_spatial_dim = (targets_spatial_dim + 1) if targets_spatial_dim is not None else Dim(None, name="blank-durations")
    if out_spatial_dim.is_dynamic() and out_spatial_dim.derived_from_op is None:
        out_spatial_dim.dyn_size_ext = Tensor("durs:size", dims=[bd[0]], dtype="int32", raw_tensor=torch.tensor([len(d) for d in out], dtype=torch.int32))
    return wrap(res.to(path._raw_tensor.device), [bd[0], out_spatial_dim]), out_spatial_dim


def ctc_greedy_decode(logits: Tensor, *, in_spatial_dim: Dim, blank_index: int, out_spatial_dim: Optional[Dim] = None,
                      target_dim: Optional[Dim] = None, wb_target_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim]:
    """
    argmax per frame, collapse repeats, remove blanks.

    :return: labels [B, out_spatial_dim] (sparse over target_dim), out_spatial_dim
    """
    from .reduce import reduce_argmax
    from .array_ import masked_select, shift_right, where
    from .math_ import logical_and

    if wb_target_dim is None:
        assert logits.feature_dim
        wb_target_dim = logits.feature_dim
    labels = reduce_argmax(logits, axis=wb_target_dim)
    labels_shifted = shift_right(labels, axis=in_spatial_dim, pad_value=blank_index)
    mask_repeat = labels != labels_shifted
    mask = logical_and(mask_repeat, labels != blank_index)
    seq_mask = in_spatial_dim.get_mask(device=labels.device) if in_spatial_dim.is_dynamic() and in_spatial_dim.is_dynamic_seq_length() else None
    if seq_mask is not None:
        mask = logical_and(mask, seq_mask)
    bd = [d for d in labels._dims if d != in_spatial_dim]
    assert len(bd) == 1
    mraw = mask.copy_compatible_to_dims_raw([bd[0], in_spatial_dim])
    lraw = labels.copy_compatible_to_dims_raw([bd[0], in_spatial_dim])
    out_lens = mraw.sum(dim=1).to(torch.int32)
    max_len = int(out_lens.max()) if out_lens.numel() else 0
    # stable partition: positions of kept labels first
    order = torch.argsort((~mraw).to(torch.int8), dim=1, stable=True)[:, :max_len]
    out = torch.gather(lraw, 1, order)
    valid = torch.arange(max_len, device=out.device)[None, :] < out_lens[:, None]
    out = torch.where(valid, out, torch.zeros_like(out))
    if out_spatial_dim is None:
        out_spatial_dim = Dim(None, name="ctc-greedy-out")
    out_spatial_dim.dyn_size_ext = Tensor("ctc-greedy:size", dims=[bd[0]], dtype="int32", raw_tensor=out_lens.cpu())
    if target_dim is not None and blank_index == target_dim.dimension:
        sparse = target_dim
    elif target_dim is not None:
        # blank inside the label set: shift labels above blank down by one
        out = torch.where(out > blank_index, out - 1, out)
        sparse = target_dim
    else:
        sparse = wb_target_dim
    return wrap(out, [bd[0], out_spatial_dim], sparse_dim=sparse), out_spatial_dim


def edit_distance(a: Tensor, a_spatial_dim: Dim, b: Tensor, b_spatial_dim: Dim, *, dtype: str = "int32") -> Tensor:
    """Levenshtein distance per batch entry: [B]"""
    from .. import native_op

    bd = [d for d in a._dims if d != a_spatial_dim]
    assert len(bd) == 1
    araw = a.copy_compatible_to_dims_raw([bd[0], a_spatial_dim])
    braw = b.copy_compatible_to_dims_raw([bd[0], b_spatial_dim])
    a_lens = _lens(a_spatial_dim, araw.shape[0], araw.shape[1])
    b_lens = _lens(b_spatial_dim, braw.shape[0], braw.shape[1])
    res = native_op.edit_distance(araw, a_lens, braw, b_lens)
    from ._utils import torch_dtype

    return wrap(res.to(torch_dtype(dtype)), [bd[0]])
