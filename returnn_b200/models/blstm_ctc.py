"""
BLSTM-CTC acoustic model: N bidirectional LSTM layers (two ``rf.LSTM`` per layer, the backward one with
``direction=-1``), optional 2x max-pool time reduction after chosen layers, linear output over vocab + blank, CTC loss.
The same file serves the small 12AX model (2 layers of 100 units, per-frame cross entropy).

    from returnn_b200.models import blstm_ctc
    get_model = blstm_ctc.get_model;  train_step = blstm_ctc.train_step

``model_opts``: ``num_layers`` (6), ``hidden`` (1024), ``in_dim`` (80), ``vocab`` (10000), ``time_reduction_after`` ((0, 1):
pool after the first two layers), ``dropout`` (0.0), ``loss`` ("ctc" | "ce": framewise cross entropy without blank).

On B200 every direction runs through the LSTM recurrence executor of :mod:`returnn_b200.ops.lstm_native`
(input projection and recurrent projections on the tcgen05 GEMM); the reference runs cuDNN here
(returnn/torch/frontend/_backend.py:2796-2810), the cell math is NativeLstm2's (returnn/native_op.py:1029).
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Sequence, Tuple
import torch
from .. import frontend as rf
from ..tensor import Tensor, Dim, TensorDict, batch_dim

DEFAULTS = dict(num_layers=6, hidden=1024, in_dim=80, vocab=10000, time_reduction_after=(0, 1), dropout=0.0, loss="ctc")


def make_extern_data(opts: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """features + labels (label sequence for CTC, framewise labels for ``loss="ce"``)"""
    o = dict(DEFAULTS, **(opts or {}))
    time_dim = Dim(None, name="time", kind=Dim.Types.Spatial)
    feat_dim = Dim(o["in_dim"], name="feature", kind=Dim.Types.Feature)
    vocab_dim = Dim(o["vocab"], name="vocab", kind=Dim.Types.Feature)
    tgt_time = time_dim if o["loss"] == "ce" else Dim(None, name="targets-time", kind=Dim.Types.Spatial)
    return {"data": {"dims": (batch_dim, time_dim, feat_dim), "dtype": "float32"},
            "classes": {"dims": (batch_dim, tgt_time), "sparse_dim": vocab_dim, "dtype": "int32", "available_for_inference": False}}


class BlstmLayer(rf.Module):
    """forward + backward LSTM, outputs concatenated"""

    def __init__(self, in_dim: Dim, hidden: Dim):
        super().__init__()
        self.fw = rf.LSTM(in_dim, hidden)
        self.bw = rf.LSTM(in_dim, hidden)
        self.out_dim = hidden + hidden

    def __call__(self, x: Tensor, *, spatial_dim: Dim) -> Tensor:
        yf, yb, _, _ = rf.bidirectional_lstm(self.fw, self.bw, x, spatial_dim=spatial_dim)
        out, _ = rf.concat((yf, self.fw.out_dim), (yb, self.bw.out_dim), out_dim=self.out_dim)
        return out


class BlstmCtcModel(rf.Module):
    """stack of BLSTM layers + output layer"""

    def __init__(self, *, in_dim: Dim, vocab_dim: Dim, num_layers: int = 6, hidden: int = 1024, time_reduction_after: Sequence[int] = (0, 1),
                 dropout: float = 0.0, loss: str = "ctc"):
        super().__init__()
        self.in_dim, self.vocab_dim, self.loss_type = in_dim, vocab_dim, loss
        self.out_vocab_dim = vocab_dim + 1 if loss == "ctc" else vocab_dim
        self.blank_idx = vocab_dim.dimension
        self.dropout = dropout
        self.time_reduction_after = tuple(time_reduction_after)
        layers = []
        cur = in_dim
        for i in range(num_layers):
            layer = BlstmLayer(cur, Dim(hidden, name="lstm%i" % i))
            layers.append(layer)
            cur = layer.out_dim
        self.layers = rf.ModuleList(*layers)
        self.output = rf.Linear(cur, self.out_vocab_dim)

    def __call__(self, source: Tensor, *, in_spatial_dim: Dim) -> Tuple[Tensor, Dim]:
        x, spatial = source, in_spatial_dim
        for i, layer in enumerate(self.layers):
            x = layer(x, spatial_dim=spatial)
            if i in self.time_reduction_after:
                x, spatial = rf.max_pool1d(x, pool_size=2, padding="same", in_spatial_dim=spatial)
            if self.dropout:
                x = rf.dropout(x, self.dropout, axis=x.feature_dim)
        return self.output(x), spatial


def get_model(*, epoch: int = 1, step: int = 0, **_kwargs) -> BlstmCtcModel:
    """config hook"""
    from ..config import get_global_config

    config = get_global_config(return_empty_if_none=True)
    opts = dict(DEFAULTS, **(config.typed_value("model_opts", None) or {}))
    extern_data = config.typed_value("extern_data")
    if extern_data:
        in_dim = extern_data["data"]["dims"][-1]
        vocab_dim = extern_data["classes"]["sparse_dim"]
    else:
        in_dim, vocab_dim = Dim(opts["in_dim"], name="feature"), Dim(opts["vocab"], name="vocab")
    return BlstmCtcModel(in_dim=in_dim, vocab_dim=vocab_dim, num_layers=opts["num_layers"], hidden=opts["hidden"],
                         time_reduction_after=opts["time_reduction_after"], dropout=opts["dropout"], loss=opts["loss"])


def train_step(*, model: BlstmCtcModel, extern_data: TensorDict, **_kwargs):
    """CTC (or framewise cross entropy + frame error rate)"""
    data, targets = extern_data["data"], extern_data["classes"]
    in_spatial_dim = data.dims[1]
    logits, enc_spatial = model(data, in_spatial_dim=in_spatial_dim)
    if model.loss_type == "ctc":
        tgt_spatial = targets.dims[1]
        loss = rf.ctc_loss(logits=logits, targets=targets, input_spatial_dim=enc_spatial, targets_spatial_dim=tgt_spatial, blank_index=model.blank_idx)
        loss.mark_as_loss("ctc", custom_inv_norm_factor=tgt_spatial.get_size_tensor(), use_normalized_loss=False)
    else:
        loss = rf.cross_entropy(estimated=logits, estimated_type="logits", target=targets, axis=model.out_vocab_dim)
        loss.mark_as_loss("ce")
        err = rf.reduce_argmax(logits, axis=model.out_vocab_dim) != targets
        err.mark_as_loss("fer", as_error=True)


def forward_step(*, model: BlstmCtcModel, extern_data: TensorDict, **_kwargs):
    """greedy decoding (CTC) or framewise posteriors"""
    data = extern_data["data"]
    logits, enc_spatial = model(data, in_spatial_dim=data.dims[1])
    if model.loss_type == "ctc":
        labels, out_dim = rf.ctc_greedy_decode(logits, in_spatial_dim=enc_spatial, blank_index=model.blank_idx, target_dim=model.vocab_dim,
                                               wb_target_dim=model.out_vocab_dim)
        rf.get_run_ctx().mark_as_output(labels, "output", dims=[batch_dim, out_dim])
    else:
        rf.get_run_ctx().mark_as_output(rf.softmax(logits, axis=model.out_vocab_dim), "output")
