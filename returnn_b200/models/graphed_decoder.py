"""
Teacher-forced ``TransformerDecoder`` + label-smoothed cross entropy as ONE pair of CUDA graphs (forward, backward) inside an
otherwise eager train step.

The decoder of an attention-based encoder-decoder model works on a few thousand tokens per step: its kernels take microseconds,
the Python that issues them milliseconds (about 8 of the 25 ms of the Conformer-AED step). The encoder of that step cannot be
captured together with it, because the packed encoder path takes its row layout from host-side lengths. So the step is
partitioned: the encoder runs as it does, its padded output is copied into a bound-shaped buffer, and the decoder + loss run as a
graphed callable (``torch.cuda.make_graphed_callables``: forward and backward captured separately and tied into autograd, so the
gradient flows back into the encoder output and the decoder's parameter gradients arrive in ``param.grad`` as usual).

Inside the captured region everything is bound-shaped: ``[batch_size_bound, capacity, ...]`` tensors, lengths in device buffers (the
masks are computed on the device, ``Dim.capacity`` is the extent), unused rows have target length 0 and are masked out of the loss.

Parity: the fw/bw partition of returnn/torch/util/graph_capture.py (``GraphCapturedTrainStep`` :410, capture with partition :1388),
here as a model-level building block.
"""

from __future__ import annotations
from typing import Optional, Tuple
import torch

from ..tensor import Tensor, Dim, batch_dim
from .. import frontend as rf


class _Body(torch.nn.Module):
    """what is captured: bound-shaped raw tensors in, (summed CE, number of wrong labels) out"""

    def __init__(self, owner: "GraphedDecoderLoss"):
        super().__init__()
        self.owner = owner
        from ..torch.frontend.bridge import rf_module_to_pt_module

        self.decoder_pt = rf_module_to_pt_module(owner.decoder)  # registers the decoder's parameters with this module

    def forward(self, enc: torch.Tensor, enc_lens: torch.Tensor, targets: torch.Tensor, tgt_lens: torch.Tensor, row_valid: torch.Tensor):
        o = self.owner
        saved_batch = batch_dim.dyn_size_ext
        try:
            with torch.autocast("cuda", dtype=o.amp_dtype, enabled=o.amp_dtype is not None, cache_enabled=False):
                batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(o.batch_bound, dtype=torch.int32))
                o.enc_spatial.dyn_size_ext = Tensor("enc-lens", dims=[batch_dim], dtype="int32", raw_tensor=enc_lens)
                o.tgt_spatial.dyn_size_ext = Tensor("tgt-lens", dims=[batch_dim], dtype="int32", raw_tensor=tgt_lens)
                enc_t = Tensor("enc", dims=[batch_dim, o.enc_spatial, o.enc_dim], dtype=str(enc.dtype).split(".")[-1], raw_tensor=enc, feature_dim=o.enc_dim)
                tgt_t = Tensor("classes", dims=[batch_dim, o.tgt_spatial], dtype=str(targets.dtype).split(".")[-1], sparse_dim=o.vocab_dim,
                               raw_tensor=targets)
                dec = o.decoder
                inp, (tgt_ext,) = rf.pad(tgt_t, axes=[o.tgt_spatial], padding=[(1, 0)], value=o.bos)
                out_t, _ = rf.pad(tgt_t, axes=[o.tgt_spatial], padding=[(0, 1)], value=o.eos, out_dims=[tgt_ext], handle_dynamic_dims=True)
                enc_state = dec.transform_encoder(enc_t, axis=o.enc_spatial)
                logits, _ = dec(inp, spatial_dim=tgt_ext, encoder=enc_state, state=dec.default_initial_state(batch_dims=[batch_dim]))
                ce, best = rf.softmax_cross_entropy_smoothed_grad(logits=logits, target=out_t, axis=o.vocab_dim, smoothing=o.label_smoothing,
                                                                  with_argmax=True)
                # frames beyond a sequence's length and the unused rows of the bound-shaped batch do not count
                frame_ok = rf.sequence_mask([batch_dim, tgt_ext]).copy_compatible_to_dims_raw([batch_dim, tgt_ext]) & (row_valid > 0)[:, None]
                ce_raw = ce.copy_compatible_to_dims_raw([batch_dim, tgt_ext]).float()
                zero = torch.zeros((), dtype=ce_raw.dtype, device=ce_raw.device)
                ce_sum = torch.where(frame_ok, ce_raw, zero).sum()
                wrong = (best.copy_compatible_to_dims_raw([batch_dim, tgt_ext]) != out_t.copy_compatible_to_dims_raw([batch_dim, tgt_ext])) & frame_ok
                return ce_sum, wrong.sum().to(torch.float32)
        finally:
            batch_dim.dyn_size_ext = saved_batch


class GraphedDecoderLoss:
    """
    :param decoder: ``rf`` ``TransformerDecoder``
    :param vocab_dim, bos, eos, label_smoothing: as in the eager formulation (input = BOS + targets, target = targets + EOS)
    :param batch_bound: sequences per batch the buffers hold
    :param enc_capacity: encoder frames per sequence
    :param tgt_capacity: target labels per sequence (without EOS)

    Call it with the padded encoder output and the targets of a batch that fits the bounds (:meth:`fits`); it returns device scalars.
    The first call warms up and captures (four eager executions of the decoder on the side stream of the capture).
    """

    def __init__(self, decoder, *, vocab_dim: Dim, enc_dim: Dim, bos: int, eos: int, label_smoothing: float, batch_bound: int, enc_capacity: int,
                 tgt_capacity: int):
        self.decoder = decoder
        self.vocab_dim, self.enc_dim = vocab_dim, enc_dim
        self.bos, self.eos, self.label_smoothing = bos, eos, label_smoothing
        self.batch_bound, self.enc_capacity, self.tgt_capacity = int(batch_bound), int(enc_capacity), int(tgt_capacity)
        self.enc_spatial = Dim(None, name="enc-time:bound", capacity=self.enc_capacity)
        self.tgt_spatial = Dim(None, name="tgt-time:bound", capacity=self.tgt_capacity)
        self.amp_dtype: Optional[torch.dtype] = None
        self._body: Optional[_Body] = None
        self._graphed = None
        self.num_replays = 0

    def fits(self, batch: int, enc_len: int, tgt_len: int) -> bool:
        """whether a batch of these extents can go through the captured graphs"""
        return batch <= self.batch_bound and enc_len <= self.enc_capacity and tgt_len <= self.tgt_capacity

    def _bound(self, enc: torch.Tensor, enc_lens: torch.Tensor, targets: torch.Tensor, tgt_lens: torch.Tensor):
        """pad to the bounds; unused rows get one encoder frame (of zeros) and no target"""
        B, T, _ = enc.shape
        S = targets.shape[1]
        dev = enc.device
        F = torch.nn.functional
        enc_b = F.pad(enc, (0, 0, 0, self.enc_capacity - T, 0, self.batch_bound - B))
        tgt_b = F.pad(targets, (0, self.tgt_capacity - S, 0, self.batch_bound - B))
        # the lengths come from the host (they are data of the batch): pinned staging, one small copy each
        el = torch.ones(self.batch_bound, dtype=torch.int32)
        el[:B] = enc_lens.to(torch.int32).cpu()
        tl = torch.zeros(self.batch_bound, dtype=torch.int32)
        tl[:B] = tgt_lens.to(torch.int32).cpu()
        valid = torch.zeros(self.batch_bound, dtype=torch.int32)
        valid[:B] = 1
        stage = torch.stack([el, tl, valid]).pin_memory().to(dev, non_blocking=True)
        return enc_b, stage[0], tgt_b, stage[1], stage[2]

    def __call__(self, enc: torch.Tensor, enc_lens: torch.Tensor, targets: torch.Tensor, tgt_lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """
        :param enc: [B, T, D] on the GPU (gradient flows back into it)
        :param enc_lens, tgt_lens: [B] lengths (host or device)
        :param targets: [B, S] labels
        :return: summed cross entropy over the valid target frames (differentiable), number of wrong arg-max labels
        """
        assert enc.is_cuda and self.fits(enc.shape[0], enc.shape[1], targets.shape[1])
        args = self._bound(enc, enc_lens, targets, tgt_lens)
        if self._graphed is None:
            self.amp_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else None
            self._body = _Body(self)
            sample = tuple(a.detach().clone().requires_grad_(a.is_floating_point()) for a in args)
            # warm-up and capture run the decoder eagerly a few times: the dropout counters advance, the losses marked meanwhile
            # belong to nobody (nothing is marked inside the body)
            with torch.autocast("cuda", enabled=False):  # the body switches autocast on itself, with the weight-cast cache off as capture wants it
                self._graphed = torch.cuda.make_graphed_callables(self._body, sample, num_warmup_iters=2, allow_unused_input=True)
        self.num_replays += 1
        with torch.autocast("cuda", enabled=False):
            return self._graphed(*args)
