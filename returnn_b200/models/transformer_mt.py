"""
Transformer-base machine translation: ``TransformerEncoder`` + ``TransformerDecoder`` (6 + 6 layers, d_model 512, 8 heads,
FFN 2048) over a shared vocabulary, label-smoothed cross entropy, beam search for translation.

    from returnn_b200.models import transformer_mt
    get_model = transformer_mt.get_model;  train_step = transformer_mt.train_step;  forward_step = transformer_mt.forward_step

``model_opts``: ``vocab`` (32000), ``model_dim`` (512), ``num_heads`` (8), ``ff_dim`` (2048), ``enc_layers`` / ``dec_layers`` (6),
``dropout`` (0.1), ``label_smoothing`` (0.1), ``beam_size`` (12), ``bos`` / ``eos`` (0), ``max_len_factor`` (1.5).
Reference building blocks: returnn/frontend/encoder/transformer.py, returnn/frontend/decoder/transformer.py.
"""

from __future__ import annotations
from typing import Any, Dict, Optional
import torch
from .. import frontend as rf
from ..tensor import Tensor, Dim, TensorDict, batch_dim
from ..frontend.encoder.transformer import TransformerEncoder
from ..frontend.decoder.transformer import TransformerDecoder
from .beam_search import beam_search_raw

DEFAULTS = dict(vocab=32000, model_dim=512, num_heads=8, ff_dim=2048, enc_layers=6, dec_layers=6, dropout=0.1, label_smoothing=0.1, beam_size=12,
                bos=0, eos=0, max_len_factor=1.5)


def make_extern_data(opts: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """source tokens ``data`` and target tokens ``classes`` over one shared vocabulary"""
    o = dict(DEFAULTS, **(opts or {}))
    vocab = Dim(o["vocab"], name="vocab", kind=Dim.Types.Feature)
    return {"data": {"dims": (batch_dim, Dim(None, name="src-time", kind=Dim.Types.Spatial)), "sparse_dim": vocab, "dtype": "int32"},
            "classes": {"dims": (batch_dim, Dim(None, name="tgt-time", kind=Dim.Types.Spatial)), "sparse_dim": vocab, "dtype": "int32",
                        "available_for_inference": False}}


class TransformerMtModel(rf.Module):
    """encoder-decoder over token ids"""

    def __init__(self, *, vocab_dim: Dim, model_dim: int = 512, num_heads: int = 8, ff_dim: int = 2048, enc_layers: int = 6, dec_layers: int = 6,
                 dropout: float = 0.1, label_smoothing: float = 0.1, beam_size: int = 12, bos: int = 0, eos: int = 0, max_len_factor: float = 1.5):
        super().__init__()
        self.vocab_dim = vocab_dim
        md = Dim(model_dim, name="model")
        self.encoder = TransformerEncoder(vocab_dim, md, num_layers=enc_layers, num_heads=num_heads, ff_dim=Dim(ff_dim, name="enc-ff"), dropout=dropout,
                                          att_dropout=dropout)
        self.decoder = TransformerDecoder(md, vocab_dim, Dim(model_dim, name="dec-model"), num_layers=dec_layers, num_heads=num_heads,
                                          ff_dim=Dim(ff_dim, name="dec-ff"), dropout=dropout, att_dropout=dropout, share_embedding=True)
        self.model_dim = md
        self.label_smoothing, self.beam_size, self.bos, self.eos, self.max_len_factor = label_smoothing, beam_size, bos, eos, max_len_factor


def get_model(*, epoch: int = 1, step: int = 0, **_kwargs) -> TransformerMtModel:
    """config hook"""
    from ..config import get_global_config

    config = get_global_config(return_empty_if_none=True)
    opts = dict(DEFAULTS, **(config.typed_value("model_opts", None) or {}))
    extern_data = config.typed_value("extern_data")
    vocab_dim = extern_data["data"]["sparse_dim"] if extern_data else Dim(opts["vocab"], name="vocab")
    return TransformerMtModel(vocab_dim=vocab_dim, **{k: opts[k] for k in DEFAULTS if k != "vocab"})


def train_step(*, model: TransformerMtModel, extern_data: TensorDict, **_kwargs):
    """teacher-forced cross entropy with label smoothing"""
    src, tgt = extern_data["data"], extern_data["classes"]
    src_spatial, tgt_spatial = src.dims[1], tgt.dims[1]
    enc = model.encoder(src, spatial_dim=src_spatial)
    inp, (tgt_ext,) = rf.pad(tgt, axes=[tgt_spatial], padding=[(1, 0)], value=model.bos)
    out_t, _ = rf.pad(tgt, axes=[tgt_spatial], padding=[(0, 1)], value=model.eos, out_dims=[tgt_ext], handle_dynamic_dims=True)
    enc_state = model.decoder.transform_encoder(enc, axis=src_spatial)
    logits, _ = model.decoder(inp, spatial_dim=tgt_ext, encoder=enc_state, state=model.decoder.default_initial_state(batch_dims=[batch_dim]))
    ce, best = rf.softmax_cross_entropy_smoothed_grad(logits=logits, target=out_t, axis=model.vocab_dim, smoothing=model.label_smoothing,
                                                      with_argmax=True)
    ce.mark_as_loss("ce", use_normalized_loss=True)
    err = best != out_t
    err.mark_as_loss("fer", as_error=True)


def forward_step(*, model: TransformerMtModel, extern_data: TensorDict, **_kwargs):
    """beam search translation: "output" = best hypothesis, "scores" = all beams"""
    from ..frontend import nested as _nested

    src = extern_data["data"]
    src_spatial = src.dims[1]
    enc = model.encoder(src, spatial_dim=src_spatial)
    B = src.raw_tensor.shape[0]
    beam, dev = model.beam_size, src.raw_tensor.device
    bb = Dim(None, name="batch-beam")
    bb.dyn_size_ext = Tensor("bb", dims=[], dtype="int32", raw_tensor=torch.tensor(B * beam, dtype=torch.int32))
    enc_bt = enc.copy_transpose([batch_dim, src_spatial, enc.feature_dim])
    sp_b = Dim(None, name="src-time-beam")
    sp_b.dyn_size_ext = Tensor("l", dims=[bb], dtype="int32", raw_tensor=src_spatial.dyn_size_ext.raw_tensor.repeat_interleave(beam))
    enc_b = Tensor("enc", dims=[bb, sp_b, enc.feature_dim], dtype=enc.dtype, raw_tensor=enc_bt.raw_tensor.repeat_interleave(beam, dim=0),
                   feature_dim=enc.feature_dim)
    dec = model.decoder
    enc_state = dec.transform_encoder(enc_b, axis=sp_b)

    def step_fn(prev, st):
        lab = Tensor("prev", dims=[bb], dtype="int64", sparse_dim=model.vocab_dim, raw_tensor=prev)
        logits, st = dec(lab, spatial_dim=rf.single_step_dim, encoder=enc_state, state=st)
        return logits.copy_transpose([bb, model.vocab_dim]).raw_tensor, st

    def reorder(st, flat):
        def g(t):
            if isinstance(t, Tensor) and t.raw_tensor is not None and bb in t.dims:
                return rf._utils.wrap(t.raw_tensor.index_select(list(t.dims).index(bb), flat), t.dims, like=t)
            return t

        return _nested.tree_map(g, st)

    max_len = torch.clamp((src_spatial.dyn_size_ext.raw_tensor.float() * model.max_len_factor).ceil().to(torch.int64), min=1)
    labels, lens, scores = beam_search_raw(step_fn, dec.default_initial_state(batch_dims=[bb]), reorder, batch=B, beam=beam, vocab=model.vocab_dim.dimension,
                                           bos=model.bos, eos=model.eos, max_len=max_len, device=dev)
    out_spatial = Dim(None, name="out-time")
    out_spatial.dyn_size_ext = Tensor("out-lens", dims=[batch_dim], dtype="int32", raw_tensor=lens[:, 0].cpu().to(torch.int32))
    best = Tensor("output", dims=[batch_dim, out_spatial], dtype="int32", sparse_dim=model.vocab_dim, raw_tensor=labels[:, 0, : int(lens[:, 0].max())])
    rf.get_run_ctx().mark_as_output(best, "output", dims=[batch_dim, out_spatial])
    rf.get_run_ctx().mark_as_output(Tensor("scores", dims=[batch_dim, Dim(beam, name="beam")], dtype="float32", raw_tensor=scores), "scores")
