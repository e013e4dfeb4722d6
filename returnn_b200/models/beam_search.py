"""
Label-synchronous beam search over any decoder with the RF step interface
(``logits, state = decoder(prev_label, spatial_dim=single_step_dim, encoder=..., state=...)``).

Per step: the decoder scores ``[batch * beam]`` hypotheses, :func:`returnn_b200.ops.seq_ops.beam_topk` does log-softmax +
score accumulation + top-k over ``beam x vocab`` + backref/label split in one kernel, then the recurrent state is gathered
by the backrefs. Finished hypotheses keep their score (optionally length-normalised at the end) and only extend with EOS.
Pattern of the reference's demo (demos/demo-rf-pt-benchmark.py:410-474) and ``rf.top_k`` (returnn/torch/frontend/_backend.py:1905-1971).
"""

from __future__ import annotations
from typing import Any, Callable, Optional, Tuple
import torch
from .. import frontend as rf
from ..tensor import Tensor, Dim, batch_dim
from ..ops import seq_ops


def beam_search_raw(step_fn: Callable[[torch.Tensor, Any], Tuple[torch.Tensor, Any]], init_state: Any,
                    reorder_state: Callable[[Any, torch.Tensor], Any], *, batch: int, beam: int, vocab: int, bos: int, eos: int,
                    max_len: torch.Tensor, device, length_norm: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    Framework-agnostic core on raw torch tensors.

    :param step_fn: ``(prev_labels [batch*beam] int64, state) -> (logits [batch*beam, vocab], state)``
    :param reorder_state: ``(state, flat_index [batch*beam]) -> state`` gathers hypotheses
    :param max_len: [batch] maximum output length per sequence (int tensor on the host)
    :return: (labels [batch, beam, L] int32 padded with eos, lengths [batch, beam], scores [batch, beam]) sorted by score
    """
    max_steps = int(max_len.max()) if batch else 0
    max_len_dev = max_len.to(device)
    scores = torch.full((batch, beam), float("-inf"), device=device)
    scores[:, 0] = 0.0  # only the first hypothesis is live at the start
    finished = torch.zeros(batch, beam, dtype=torch.bool, device=device)
    lengths = torch.zeros(batch, beam, dtype=torch.int32, device=device)
    prev = torch.full((batch * beam,), bos, dtype=torch.int64, device=device)
    state = init_state
    hist_labels, hist_back = [], []
    for i in range(max_steps):
        logits, state = step_fn(prev, state)
        logits = logits.reshape(batch, beam, vocab)
        # hypotheses that reached their length limit may only end
        force_end = (lengths >= (max_len_dev[:, None] - 1)) & ~finished
        if bool(force_end.any()):
            forced = torch.full_like(logits, float("-inf"))
            forced[..., eos] = 0.0
            logits = torch.where(force_end[..., None], forced.to(logits.dtype), logits)
        new_scores, back, lab = seq_ops.beam_topk(logits, scores, finished=finished, eos=eos, k=beam)
        flat = (torch.arange(batch, device=device)[:, None] * beam + back.long()).reshape(-1)
        state = reorder_state(state, flat)
        was_finished = finished.reshape(-1)[flat].reshape(batch, beam)
        lengths = lengths.reshape(-1)[flat].reshape(batch, beam) + (~was_finished).to(torch.int32)
        finished = was_finished | (lab == eos)
        scores = new_scores
        hist_labels.append(lab)
        hist_back.append(back)
        prev = lab.reshape(-1).long()
        if bool(finished.all()):
            break
    # backtrace
    L = len(hist_labels)
    out = torch.full((batch, beam, max(L, 1)), eos, dtype=torch.int32, device=device)
    idx = torch.arange(beam, device=device)[None, :].expand(batch, beam)
    for i in range(L - 1, -1, -1):
        out[:, :, i] = torch.gather(hist_labels[i], 1, idx)
        idx = torch.gather(hist_back[i].long(), 1, idx)
    final = scores
    if length_norm:
        final = scores / torch.clamp(lengths.float(), min=1.0)
    order = torch.argsort(final, dim=1, descending=True)
    return (torch.gather(out, 1, order[:, :, None].expand_as(out)), torch.gather(lengths, 1, order), torch.gather(final, 1, order))
