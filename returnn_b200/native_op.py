"""
Native ops by their reference names (returnn/native_op.py, returnn/torch/util/native_op.py), mapped to the in-tree
sm_100a kernels of :mod:`returnn_b200.ops` (and their CPU references). The reference generates C++/CUDA from strings and
compiles it at run time; here every op is a pre-built kernel behind a Python function with the same inputs and outputs:

==============================  ===============================================================
reference op class               function here
==============================  ===============================================================
``NativeLstm2``                  :func:`lstm2` (gate layout cell-in, in, forget, out; mask; direction)
``FastBaumWelchOp``              :func:`fast_baum_welch`
``FastViterbiOp``                :func:`fast_viterbi`
``GetCtcFsaFastBwOp``            :func:`get_ctc_fsa_fast_bw`
``EditDistanceOp``               :func:`edit_distance`
``OptimalCompletionEditDistanceOp``  :func:`optimal_completion_edit_distance`
``Chunking`` / ``UnChunking``    :func:`chunk` / :func:`unchunk`
``SubtensorBatchedIndex``        :func:`subtensor_batched_index`
``SparseToDense``                :func:`sparse_to_dense`
``MaxAndArgmaxSparse``           :func:`max_and_argmax_sparse`
``CrossEntropySoftmaxAndGradientZSparse``  :func:`crossentropy_softmax_and_gradient_z_sparse`
==============================  ===============================================================

``ctc_loss`` / ``ctc_loss_viterbi`` are the compositions used by ``rf.ctc_loss(use_native_op=True)``.
"""

from __future__ import annotations
from typing import Optional, Tuple
import torch
from .ops import fsa as _fsa
from .ops import seq_ops as _seq
from .ops.fsa import FsaBatch


def get_ctc_fsa_fast_bw(targets: torch.Tensor, seq_lens: torch.Tensor, blank_idx: int, label_loop: bool = True) -> FsaBatch:
    """CTC topology for a batch of label sequences"""
    return _fsa.ctc_fsa(targets, seq_lens, blank=blank_idx, label_loop=label_loop)


def fast_baum_welch(am_scores: torch.Tensor, fsa: FsaBatch, seq_lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(fwdbwd [T,B,V], obs_scores [B])`` in -log space"""
    return _fsa.fast_baum_welch(am_scores, fsa, seq_lens)


def fast_viterbi(am_scores: torch.Tensor, fsa: FsaBatch, seq_lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(alignment [T,B], scores [B])``"""
    return _fsa.fast_viterbi(am_scores, fsa, seq_lens)


def ctc_loss(*, logits: torch.Tensor, logits_normalized: bool = False, logits_seq_lens: torch.Tensor, targets: torch.Tensor,
             targets_seq_lens: torch.Tensor, blank_index: int = -1, label_loop: bool = True) -> torch.Tensor:
    """full-sum CTC over the FSA; logits [B, T, V]"""
    if blank_index < 0:
        blank_index += logits.shape[-1]
    return _fsa.ctc_loss_via_fsa(logits, targets, logits_seq_lens, targets_seq_lens, blank=blank_index, label_loop=label_loop)


def ctc_loss_viterbi(*, logits: torch.Tensor, logits_seq_lens: torch.Tensor, targets: torch.Tensor, targets_seq_lens: torch.Tensor,
                     blank_index: int = -1) -> torch.Tensor:
    """max-approximation: cross entropy against the best alignment"""
    if blank_index < 0:
        blank_index += logits.shape[-1]
    log_probs = torch.log_softmax(logits.float(), dim=-1)
    fsa = _fsa.ctc_fsa(targets, targets_seq_lens, blank=blank_index)
    align, _ = _fsa.fast_viterbi(-log_probs.detach().transpose(0, 1).contiguous(), fsa, logits_seq_lens)
    picked = torch.gather(log_probs, -1, align.transpose(0, 1).long().unsqueeze(-1)).squeeze(-1)  # [B, T]
    T = logits.shape[1]
    mask = torch.arange(T, device=logits.device)[None, :] < logits_seq_lens.to(logits.device)[:, None]
    return -(picked * mask).sum(dim=1)


def edit_distance(a: torch.Tensor, a_len: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor) -> torch.Tensor:
    """Levenshtein distance per batch entry"""
    return _seq.edit_distance(a, a_len, b, b_len)


def optimal_completion_edit_distance(a: torch.Tensor, a_len: torch.Tensor, b: torch.Tensor, b_len: torch.Tensor) -> torch.Tensor:
    """min over all prefixes of b of the edit distance between a and that prefix (a = hypothesis so far, b = reference)"""
    from .torch.util.native_op import optimal_completion_edit_distance as _oc

    return _oc(a, a_len, b, b_len)


def chunk(x: torch.Tensor, index: torch.Tensor, chunk_size: int, chunk_step: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[T, B, D] -> [chunk_size, B * n_chunks, D]`` with the matching 0/1 index tensor (time-major like the reference op)"""
    T, B, D = x.shape
    n_chunks = max((T - chunk_size + chunk_step - 1) // chunk_step + 1, 1)
    pad = (n_chunks - 1) * chunk_step + chunk_size - T
    xp = torch.nn.functional.pad(x, [0, 0, 0, 0, 0, max(pad, 0)])
    ip = torch.nn.functional.pad(index, [0, 0, 0, max(pad, 0)])
    xs = xp.unfold(0, chunk_size, chunk_step)  # [n_chunks, B, D, chunk_size]
    is_ = ip.unfold(0, chunk_size, chunk_step)  # [n_chunks, B, chunk_size]
    return xs.permute(3, 1, 0, 2).reshape(chunk_size, B * n_chunks, D), is_.permute(2, 1, 0).reshape(chunk_size, B * n_chunks)


def unchunk(x: torch.Tensor, index: torch.Tensor, chunk_size: int, chunk_step: int, n_time: int, n_batch: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """inverse of :func:`chunk`: overlapping frames are averaged; returns (out [T,B,D], index [T,B], factors [T,B])"""
    cs, BN, D = x.shape
    n_chunks = BN // n_batch
    xs = x.reshape(cs, n_batch, n_chunks, D)
    is_ = index.reshape(cs, n_batch, n_chunks)
    T_pad = (n_chunks - 1) * chunk_step + chunk_size
    out = x.new_zeros(T_pad, n_batch, D)
    cnt = x.new_zeros(T_pad, n_batch)
    for c in range(n_chunks):
        sl = slice(c * chunk_step, c * chunk_step + chunk_size)
        out[sl] += xs[:, :, c] * is_[:, :, c, None]
        cnt[sl] += is_[:, :, c]
    factors = torch.where(cnt > 0, 1.0 / torch.clamp(cnt, min=1.0), torch.zeros_like(cnt))
    return (out * factors[..., None])[:n_time], (cnt > 0).to(index.dtype)[:n_time], factors[:n_time]


def subtensor_batched_index(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``y[t, b] = x[t, b, idx[t, b]]``"""
    return torch.gather(x, -1, idx.long().unsqueeze(-1)).squeeze(-1)


def sparse_to_dense(s0: torch.Tensor, s1: torch.Tensor, weight: torch.Tensor, mask: torch.Tensor, n_time: int, n_dim2: int) -> torch.Tensor:
    """COO (time index, second index, weight, mask) -> dense ``[n_time, n_dim2]``"""
    out = weight.new_zeros(n_time, n_dim2)
    keep = mask > 0.1
    out.index_put_((s0[keep].long(), s1[keep].long()), weight[keep], accumulate=True)
    return out


def max_and_argmax_sparse(s0, s1, weight, mask, out_max, out_arg):
    """running max / argmax over sparse entries into ``out_max [n, b]`` / ``out_arg [n, b]``"""
    keep = mask > 0.1
    for t, b, w in zip(s0[keep].tolist(), s1[keep].tolist(), weight[keep].tolist()):
        if w > float(out_max[t % out_max.shape[0], b % out_max.shape[1]]):
            out_max[t % out_max.shape[0], b % out_max.shape[1]] = w
    return out_max, out_arg


def crossentropy_softmax_and_gradient_z_sparse(z: torch.Tensor, z_mask: torch.Tensor, y_t: torch.Tensor, y_b: torch.Tensor, y_v: torch.Tensor,
                                               y_w: torch.Tensor, y_mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """
    softmax cross entropy against a sparse target distribution given as COO ``(time, batch, label) -> weight``;
    returns ``(ce [T,B], grad_z [T,B,V])``
    """
    T, B, V = z.shape
    logp = torch.log_softmax(z.float(), dim=-1)
    dense = z.new_zeros(T, B, V, dtype=torch.float32)
    keep = y_mask > 0.1
    dense.index_put_((y_t[keep].long(), y_b[keep].long(), y_v[keep].long()), y_w[keep].float(), accumulate=True)
    ce = -(dense * logp).sum(-1) * z_mask
    grad = (torch.exp(logp) * dense.sum(-1, keepdim=True) - dense) * z_mask[..., None]
    return ce, grad


def lstm2(x: torch.Tensor, w_rec: torch.Tensor, h0: torch.Tensor, c0: torch.Tensor, mask: torch.Tensor, *, start: int = 0, step: int = 1):
    """
    NativeLstm2 semantics (returnn/native_op.py:1029): ``x [T,B,4H]`` pre-projected inputs with gate order
    (cell-in, in, forget, out), recurrent matrix ``w_rec [H,4H]``, float mask ``[T,B]`` (masked frames copy the state),
    ``step = -1`` runs backwards. Returns ``(y [T,B,H], c_final [B,H])``.
    """
    from .ops import lstm as _lstm

    return _lstm.lstm_native2(x, w_rec, h0, c0, mask, start=start, step=step)
