"""
Conformer-CTC: ``ConformerEncoder`` (conv2d subsampling x6, N layers) + linear output layer over vocab + blank, CTC loss.

``get_model`` / ``train_step`` / ``forward_step`` here are what a config refers to:

    from returnn_b200.models import conformer_ctc
    get_model = conformer_ctc.get_model;  train_step = conformer_ctc.train_step

Model hyper-parameters come from the config dict ``model_opts``. On B200 the step runs the fused packed-row path
(:mod:`returnn_b200.models.conformer_fused`); elsewhere (or with ``model_opts["fused"] = False``) the generic RF path.
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Tuple
import torch
from .. import frontend as rf
from ..tensor import Tensor, Dim, TensorDict, batch_dim
from ..frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample
from . import conformer_fused
from .packing import PackInfo

DEFAULTS = dict(num_layers=12, model_dim=512, num_heads=8, ff_dim=2048, conv_kernel_size=32, in_dim=80, vocab=10000,
                dropout=0.1, att_dropout=0.1, conv_channels=(32, 64, 64))


def make_extern_data(opts: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """``extern_data`` for audio features + BPE labels"""
    o = dict(DEFAULTS, **(opts or {}))
    time_dim = Dim(None, name="time", kind=Dim.Types.Spatial)
    feat_dim = Dim(o["in_dim"], name="feature", kind=Dim.Types.Feature)
    targets_time = Dim(None, name="targets-time", kind=Dim.Types.Spatial)
    vocab_dim = Dim(o["vocab"], name="vocab", kind=Dim.Types.Feature)
    return {
        "data": {"dims": (batch_dim, time_dim, feat_dim), "dtype": "float32"},
        "classes": {"dims": (batch_dim, targets_time), "sparse_dim": vocab_dim, "dtype": "int32", "available_for_inference": False},
    }


class ConformerCtcModel(rf.Module):
    """encoder + output layer"""

    def __init__(self, *, in_dim: Dim, vocab_dim: Dim, num_layers: int = 12, model_dim: int = 512, num_heads: int = 8,
                 ff_dim: int = 2048, conv_kernel_size: int = 32, dropout: float = 0.1, att_dropout: float = 0.1,
                 conv_channels=(32, 64, 64), fused: Optional[bool] = None):
        super().__init__()
        self.in_dim = in_dim
        self.vocab_dim = vocab_dim
        self.wb_vocab_dim = vocab_dim + 1
        self.blank_idx = vocab_dim.dimension
        self.model_dim = Dim(model_dim, name="enc-model")
        c1, c2, c3 = conv_channels
        self.encoder = ConformerEncoder(
            in_dim, self.model_dim, num_layers=num_layers, num_heads=num_heads, ff_dim=Dim(ff_dim, name="enc-ff"),
            conv_kernel_size=conv_kernel_size, dropout=dropout, att_dropout=att_dropout,
            conv_norm=rf.build_dict(rf.BatchNorm, use_mask=True),  # statistics over valid frames: the same model on padded and on packed batches
            input_layer=ConformerConvSubsample(in_dim, out_dims=[Dim(c1, name="conv1"), Dim(c2, name="conv2"), Dim(c3, name="conv3")],
                                               filter_sizes=[(3, 3), (3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)]))
        self.logits = rf.Linear(self.model_dim, self.wb_vocab_dim)
        self.fused = fused

    def use_fused(self, x: Tensor) -> bool:
        """fused path: CUDA input, standard configuration, not disabled"""
        if self.fused is False:
            return False
        if not x.raw_tensor.is_cuda:
            return False
        return conformer_fused.supports_fused(self.encoder)

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim) -> Tuple[Tensor, Dim]:
        """generic path: logits [B, T', V+1]"""
        enc, enc_spatial_dim = self.encoder(source, in_spatial_dim=in_spatial_dim)
        return self.logits(enc), enc_spatial_dim

    def fused_logits(self, feats: torch.Tensor, lens_host: torch.Tensor, *, training: bool) -> Tuple[torch.Tensor, PackInfo]:
        """fused path: packed logits [N, V+1] in bf16"""
        from ..ops import linear as _lin

        from ..parallel import arena as _arena

        rows, pack = conformer_fused.encode_packed(self.encoder, feats, lens_host, training=training)
        w = self.logits.weight.raw_tensor
        b = self.logits.bias.raw_tensor
        ar = _arena.find_arena(w) if (training and torch.is_grad_enabled()) else None
        if ar is not None and w.shape[1] % 8:
            # vocabulary + blank is odd-sized: computed 8-aligned, the extra classes have probability 0 (the CTC loss takes
            # the number of classes from the logits)
            from ..ops import gemm as _gemm

            logits = _gemm.linear_arena_padded_out(rows, w, b, ar)
            if logits is not None:
                return logits, pack
        logits = conformer_fused.arena_linear(rows, w, b, None, ar, conformer_fused._Weights(rows.dtype))
        return logits, pack


def get_model(*, epoch: int = 1, step: int = 0, **_kwargs) -> ConformerCtcModel:
    """config hook"""
    from ..config import get_global_config

    config = get_global_config(return_empty_if_none=True)
    opts = dict(DEFAULTS, **(config.typed_value("model_opts", None) or {}))
    extern_data = config.typed_value("extern_data")
    if extern_data:
        in_dim = extern_data["data"]["dims"][-1]
        vocab_dim = extern_data["classes"]["sparse_dim"]
    else:
        in_dim = Dim(opts["in_dim"], name="feature")
        vocab_dim = Dim(opts["vocab"], name="vocab")
    return ConformerCtcModel(in_dim=in_dim, vocab_dim=vocab_dim, num_layers=opts["num_layers"], model_dim=opts["model_dim"],
                             num_heads=opts["num_heads"], ff_dim=opts["ff_dim"], conv_kernel_size=opts["conv_kernel_size"],
                             dropout=opts["dropout"], att_dropout=opts["att_dropout"], conv_channels=tuple(opts["conv_channels"]),
                             fused=opts.get("fused", None))


def train_step(*, model: ConformerCtcModel, extern_data: TensorDict, **_kwargs):
    """CTC loss, normalised by the number of target labels for reporting"""
    data = extern_data["data"]
    targets = extern_data["classes"]
    in_spatial_dim = data.dims[1]
    targets_spatial_dim = targets.dims[1]
    if model.use_fused(data):
        from ..ops import ctc as _ctc

        lens_host = in_spatial_dim.dyn_size_ext.raw_tensor
        training = bool(rf.get_run_ctx().train_flag)
        logits, pack = model.fused_logits(data.raw_tensor, lens_host, training=training)
        tgt_lens_host = targets_spatial_dim.dyn_size_ext.raw_tensor
        loss_raw = _ctc.ctc_loss_packed(logits, pack, targets.raw_tensor, tgt_lens_host, blank_index=model.blank_idx)
        loss = Tensor("ctc", dims=[batch_dim], dtype="float32", raw_tensor=loss_raw)
    else:
        logits, enc_spatial_dim = model(data, in_spatial_dim=in_spatial_dim)
        loss = rf.ctc_loss(logits=logits, targets=targets, input_spatial_dim=enc_spatial_dim, targets_spatial_dim=targets_spatial_dim,
                           blank_index=model.blank_idx)
    loss.mark_as_loss("ctc", custom_inv_norm_factor=targets_spatial_dim.get_size_tensor(), use_normalized_loss=False)


def forward_step(*, model: ConformerCtcModel, extern_data: TensorDict, **_kwargs):
    """greedy CTC decoding: output "output" = label sequence"""
    data = extern_data["data"]
    in_spatial_dim = data.dims[1]
    logits, enc_spatial_dim = model(data, in_spatial_dim=in_spatial_dim)
    labels, out_dim = rf.ctc_greedy_decode(logits, in_spatial_dim=enc_spatial_dim, blank_index=model.blank_idx, target_dim=model.vocab_dim,
                                           wb_target_dim=model.wb_vocab_dim)
    rf.get_run_ctx().mark_as_output(labels, "output", dims=[batch_dim, out_dim])
