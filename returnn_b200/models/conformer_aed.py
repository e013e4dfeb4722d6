"""
Attention encoder-decoder ASR: Conformer encoder (as in :mod:`returnn_b200.models.conformer_ctc`) + Transformer decoder
with cross-attention; loss = label-smoothed cross entropy + ``aux_ctc_scale`` x CTC on the encoder output; recognition by
beam search (:mod:`returnn_b200.models.beam_search`).

    from returnn_b200.models import conformer_aed
    get_model = conformer_aed.get_model;  train_step = conformer_aed.train_step;  forward_step = conformer_aed.forward_step

``model_opts``: encoder options of conformer_ctc plus ``dec_layers`` (6), ``label_smoothing`` (0.1), ``aux_ctc_scale`` (0.3),
``beam_size`` (12), ``max_len_factor`` (0.3: output length limit relative to the encoder length), ``bos`` / ``eos`` (0).
Reference building blocks: returnn/frontend/encoder/conformer.py, returnn/frontend/decoder/transformer.py.
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Tuple
import torch
from .. import frontend as rf
from ..tensor import Tensor, Dim, TensorDict, batch_dim
from ..frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample
from ..frontend.decoder.transformer import TransformerDecoder
from . import conformer_ctc, conformer_fused
from .beam_search import beam_search_raw

DEFAULTS = dict(conformer_ctc.DEFAULTS, dec_layers=6, label_smoothing=0.1, aux_ctc_scale=0.3, beam_size=12, max_len_factor=0.3, bos=0, eos=0)
make_extern_data = conformer_ctc.make_extern_data


class ConformerAedModel(rf.Module):
    """encoder, decoder, aux CTC output"""

    def __init__(self, *, in_dim: Dim, vocab_dim: Dim, num_layers: int = 12, model_dim: int = 512, num_heads: int = 8, ff_dim: int = 2048,
                 conv_kernel_size: int = 32, dropout: float = 0.1, att_dropout: float = 0.1, conv_channels=(32, 64, 64), dec_layers: int = 6,
                 label_smoothing: float = 0.1, aux_ctc_scale: float = 0.3, beam_size: int = 12, max_len_factor: float = 0.3, bos: int = 0, eos: int = 0,
                 graphed_decoder: Optional[dict] = None):
        """
        :param graphed_decoder: ``{"batch_size_bound", "enc_capacity", "tgt_capacity"}``: in training on the GPU the decoder and its loss run as
            a captured pair of CUDA graphs over buffers of these bounds (``models/graphed_decoder.py``); batches beyond them run eagerly
        """
        super().__init__()
        self.graphed_decoder_opts = dict(graphed_decoder) if graphed_decoder else None
        self._graphed_decoder = None
        self.in_dim, self.vocab_dim = in_dim, vocab_dim
        self.wb_vocab_dim = vocab_dim + 1
        self.blank_idx = vocab_dim.dimension
        self.model_dim = Dim(model_dim, name="enc-model")
        c1, c2, c3 = conv_channels
        self.encoder = ConformerEncoder(
            in_dim, self.model_dim, num_layers=num_layers, num_heads=num_heads, ff_dim=Dim(ff_dim, name="enc-ff"), conv_kernel_size=conv_kernel_size,
            dropout=dropout, att_dropout=att_dropout,
            conv_norm=rf.build_dict(rf.BatchNorm, use_mask=True),  # statistics over valid frames: the same model on padded and on packed batches
            input_layer=ConformerConvSubsample(in_dim, out_dims=[Dim(c1, name="conv1"), Dim(c2, name="conv2"), Dim(c3, name="conv3")],
                                               filter_sizes=[(3, 3), (3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)]))
        self.decoder = TransformerDecoder(encoder_dim=self.model_dim, vocab_dim=vocab_dim, model_dim=Dim(model_dim, name="dec-model"),
                                          num_layers=dec_layers, num_heads=num_heads, ff_dim=Dim(ff_dim, name="dec-ff"), dropout=dropout,
                                          att_dropout=att_dropout)
        self.aux_ctc = rf.Linear(self.model_dim, self.wb_vocab_dim) if aux_ctc_scale else None
        self.label_smoothing, self.aux_ctc_scale = label_smoothing, aux_ctc_scale
        self.beam_size, self.max_len_factor, self.bos, self.eos = beam_size, max_len_factor, bos, eos

    def aux_logits(self, enc: Tensor) -> Tensor:
        """
        logits of the auxiliary CTC output. The width (vocabulary + blank) is odd: in training on the GPU the layer is computed
        8-aligned on the tcgen05 GEMM with extra classes of probability 0 (the CTC loss takes the number of classes from the
        logits it gets); elsewhere the plain linear layer.
        """
        raw = enc.raw_tensor
        w = self.aux_ctc.weight.raw_tensor
        if raw.is_cuda and w.shape[1] % 8 and torch.is_grad_enabled() and raw.requires_grad:
            from ..ops import gemm as _gemm
            from ..parallel import arena as _arena

            ar = _arena.find_arena(w)
            if ar is not None and enc.dims[-1] == self.model_dim:
                out = _gemm.linear_arena_padded_out(raw.reshape(-1, raw.shape[-1]), w, self.aux_ctc.bias.raw_tensor, ar)
                if out is not None:
                    pad_dim = Dim(int(out.shape[-1]), name="vocab+blank:padded")
                    return Tensor("aux_logits", dims=list(enc.dims[:-1]) + [pad_dim], dtype=str(out.dtype).split(".")[-1],
                                  raw_tensor=out.reshape(*raw.shape[:-1], out.shape[-1]), feature_dim=pad_dim)
        return self.aux_ctc(enc)

    def encode(self, source: Tensor, *, in_spatial_dim: Dim) -> Tuple[Tensor, Dim]:
        """encoder output [B, T', D]; on B200 in training the packed native path, unpacked again for the decoder"""
        raw = source.raw_tensor
        training = bool(rf.get_run_ctx().train_flag)
        if raw.is_cuda and training and conformer_fused.supports_fused(self.encoder):
            lens_host = in_spatial_dim.dyn_size_ext.raw_tensor
            rows, pack = conformer_fused.encode_packed(self.encoder, raw, lens_host, training=True)
            padded = pack.unpack(rows)
            out_spatial = Dim(None, name="enc-time")
            out_spatial.dyn_size_ext = Tensor("enc-lens", dims=[batch_dim], dtype="int32", raw_tensor=pack.lens_host.clone())
            return Tensor("enc", dims=[batch_dim, out_spatial, self.model_dim], dtype=str(padded.dtype).split(".")[-1], raw_tensor=padded,
                          feature_dim=self.model_dim), out_spatial
        return self.encoder(source, in_spatial_dim=in_spatial_dim)


def get_model(*, epoch: int = 1, step: int = 0, **_kwargs) -> ConformerAedModel:
    """config hook"""
    from ..config import get_global_config

    config = get_global_config(return_empty_if_none=True)
    opts = dict(DEFAULTS, **(config.typed_value("model_opts", None) or {}))
    extern_data = config.typed_value("extern_data")
    if extern_data:
        in_dim, vocab_dim = extern_data["data"]["dims"][-1], extern_data["classes"]["sparse_dim"]
    else:
        in_dim, vocab_dim = Dim(opts["in_dim"], name="feature"), Dim(opts["vocab"], name="vocab")
    keys = ("num_layers", "model_dim", "num_heads", "ff_dim", "conv_kernel_size", "dropout", "att_dropout", "dec_layers", "label_smoothing",
            "aux_ctc_scale", "beam_size", "max_len_factor", "bos", "eos")
    return ConformerAedModel(in_dim=in_dim, vocab_dim=vocab_dim, conv_channels=tuple(opts["conv_channels"]), graphed_decoder=opts.get("graphed_decoder"),
                             **{k: opts[k] for k in keys})


def train_step(*, model: ConformerAedModel, extern_data: TensorDict, **_kwargs):
    """label-smoothed CE over the decoder outputs + auxiliary CTC on the encoder"""
    data, targets = extern_data["data"], extern_data["classes"]
    tgt_spatial = targets.dims[1]
    enc, enc_spatial = model.encode(data, in_spatial_dim=data.dims[1])
    if model.aux_ctc is not None:
        ctc = rf.ctc_loss(logits=model.aux_logits(enc), targets=targets, input_spatial_dim=enc_spatial, targets_spatial_dim=tgt_spatial,
                          blank_index=model.blank_idx)
        ctc.mark_as_loss("ctc", scale=model.aux_ctc_scale, custom_inv_norm_factor=tgt_spatial.get_size_tensor(), use_normalized_loss=False)
    if _graphed_decoder_loss(model, enc, enc_spatial, targets, tgt_spatial):
        return
    # teacher forcing: decoder input = BOS + targets[:-1], target = targets + EOS
    inp, (tgt_ext,) = rf.pad(targets, axes=[tgt_spatial], padding=[(1, 0)], value=model.bos)
    out_t, _ = rf.pad(targets, axes=[tgt_spatial], padding=[(0, 1)], value=model.eos, out_dims=[tgt_ext], handle_dynamic_dims=True)
    enc_state = model.decoder.transform_encoder(enc, axis=enc_spatial)
    logits, _ = model.decoder(inp, spatial_dim=tgt_ext, encoder=enc_state, state=model.decoder.default_initial_state(batch_dims=[batch_dim]))
    ce, best = rf.softmax_cross_entropy_smoothed_grad(logits=logits, target=out_t, axis=model.vocab_dim, smoothing=model.label_smoothing,
                                                      with_argmax=True)
    ce.mark_as_loss("ce", use_normalized_loss=True)
    err = best != out_t
    err.mark_as_loss("fer", as_error=True)


def _graphed_decoder_loss(model: ConformerAedModel, enc: Tensor, enc_spatial: Dim, targets: Tensor, tgt_spatial: Dim) -> bool:
    """the decoder + cross entropy through the captured graphs when configured and the batch fits; marks "ce" and "fer"; False: not taken"""
    opts = model.graphed_decoder_opts
    enc_raw = enc.copy_transpose([batch_dim, enc_spatial, model.model_dim]).raw_tensor
    if not opts or not enc_raw.is_cuda or not rf.get_run_ctx().train_flag or not torch.is_grad_enabled():
        return False
    if model._graphed_decoder is None:
        from .graphed_decoder import GraphedDecoderLoss

        model._graphed_decoder = GraphedDecoderLoss(
            model.decoder, vocab_dim=model.vocab_dim, enc_dim=model.model_dim, bos=model.bos, eos=model.eos, label_smoothing=model.label_smoothing,
            batch_bound=opts["batch_size_bound"], enc_capacity=opts["enc_capacity"], tgt_capacity=opts["tgt_capacity"])
    gd = model._graphed_decoder
    tgt_raw = targets.copy_transpose([batch_dim, tgt_spatial]).raw_tensor
    if not gd.fits(enc_raw.shape[0], enc_raw.shape[1], tgt_raw.shape[1]):
        return False
    tgt_lens = tgt_spatial.dyn_size_ext.raw_tensor
    ce_sum, wrong = gd(enc_raw, enc_spatial.dyn_size_ext.raw_tensor, tgt_raw, tgt_lens)
    n_frames = int(tgt_lens.sum()) + int(tgt_raw.shape[0])  # every sequence has its labels and the end symbol
    ctx = rf.get_run_ctx()
    ctx.mark_as_loss(Tensor("ce", dims=[], dtype="float32", raw_tensor=ce_sum), "ce", use_normalized_loss=True, custom_inv_norm_factor=n_frames)
    ctx.mark_as_loss(Tensor("fer", dims=[], dtype="float32", raw_tensor=wrong), "fer", as_error=True, custom_inv_norm_factor=n_frames)
    return True


def forward_step(*, model: ConformerAedModel, extern_data: TensorDict, **_kwargs):
    """beam search; outputs "output" (best hypothesis labels) and "scores" (all beams)"""
    data = extern_data["data"]
    enc, enc_spatial = model.encode(data, in_spatial_dim=data.dims[1])
    labels, lens, scores = recognize(model, enc, enc_spatial)
    out_spatial = Dim(None, name="out-time")
    out_spatial.dyn_size_ext = Tensor("out-lens", dims=[batch_dim], dtype="int32", raw_tensor=lens[:, 0].cpu().to(torch.int32))
    best = Tensor("output", dims=[batch_dim, out_spatial], dtype="int32", sparse_dim=model.vocab_dim, raw_tensor=labels[:, 0, : int(lens[:, 0].max())])
    rf.get_run_ctx().mark_as_output(best, "output", dims=[batch_dim, out_spatial])
    beam_dim = Dim(model.beam_size, name="beam")
    rf.get_run_ctx().mark_as_output(Tensor("scores", dims=[batch_dim, beam_dim], dtype="float32", raw_tensor=scores), "scores")


def recognize(model: ConformerAedModel, enc: Tensor, enc_spatial: Dim):
    """beam search on raw tensors: (labels [B, beam, L], lengths [B, beam], scores [B, beam])"""
    dec = model.decoder
    B = enc.raw_tensor.shape[enc.dims.index(batch_dim)]
    beam = model.beam_size
    dev = enc.raw_tensor.device
    # expand the encoder to batch*beam hypotheses
    beam_batch = Dim(None, name="batch-beam")
    beam_batch.dyn_size_ext = Tensor("bb", dims=[], dtype="int32", raw_tensor=torch.tensor(B * beam, dtype=torch.int32))
    enc_bt = enc.copy_transpose([batch_dim, enc_spatial, enc.feature_dim])
    enc_raw = enc_bt.raw_tensor.repeat_interleave(beam, dim=0)
    max_len = torch.clamp((enc_spatial.dyn_size_ext.raw_tensor.float() * model.max_len_factor).ceil().to(torch.int64), min=1)
    if getattr(model, "static_decode", True) and not torch.is_grad_enabled():
        # one CUDA-graph replay per label over static caches (models/decode_graph.py); decoders it does not cover use the loop below
        from .decode_graph import StaticTransformerDecoderStep, beam_search_static

        try:
            stepper = StaticTransformerDecoderStep(dec, enc=enc_bt.raw_tensor, enc_lens=enc_spatial.dyn_size_ext.raw_tensor,
                                                   num_hyps=B * beam, max_steps=int(max_len.max()),
                                                   dtype=torch.bfloat16 if (dev.type == "cuda" and torch.is_autocast_enabled()) else None)
        except TypeError:
            stepper = None
        if stepper is not None:
            return beam_search_static(stepper, batch=B, beam=beam, bos=model.bos, eos=model.eos, max_len=max_len)
    spatial_b = Dim(None, name="enc-time-beam")
    spatial_b.dyn_size_ext = Tensor("l", dims=[beam_batch], dtype="int32", raw_tensor=enc_spatial.dyn_size_ext.raw_tensor.repeat_interleave(beam))
    enc_b = Tensor("enc", dims=[beam_batch, spatial_b, enc.feature_dim], dtype=enc.dtype, raw_tensor=enc_raw, feature_dim=enc.feature_dim)
    enc_state = dec.transform_encoder(enc_b, axis=spatial_b)
    state = dec.default_initial_state(batch_dims=[beam_batch])

    def step_fn(prev: torch.Tensor, st):
        lab = Tensor("prev", dims=[beam_batch], dtype="int64", sparse_dim=model.vocab_dim, raw_tensor=prev)
        logits, st = dec(lab, spatial_dim=rf.single_step_dim, encoder=enc_state, state=st)
        return logits.copy_transpose([beam_batch, model.vocab_dim]).raw_tensor, st

    from ..frontend import nested as _nested

    def reorder(st, flat):
        def g(t):
            if isinstance(t, Tensor) and t.raw_tensor is not None and beam_batch in t.dims:
                ax = list(t.dims).index(beam_batch)
                return rf._utils.wrap(t.raw_tensor.index_select(ax, flat), t.dims, like=t)
            return t

        return _nested.tree_map(g, st)

    return beam_search_raw(step_fn, state, reorder, batch=B, beam=beam, vocab=model.vocab_dim.dimension, bos=model.bos, eos=model.eos,
                           max_len=max_len, device=dev)
