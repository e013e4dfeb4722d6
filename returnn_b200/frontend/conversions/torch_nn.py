"""
``torch.nn`` modules -> RF modules (reference: returnn/frontend/conversions/torch_nn.py:14, :30, :48).
Layouts: ``torch.nn.Linear.weight`` is (out, in), ``rf.Linear.weight`` is (in, out); ``torch.nn.Conv1d.weight`` and
``rf.Conv1d.filter`` are both (out, in / groups, width).
"""

from __future__ import annotations
import torch
from ..linear import Linear
from ..conv import Conv1d
from ..normalization import LayerNorm
from ._common import assign, check_same_num_params

__all__ = ["import_params_torch_linear_to_rf", "import_params_torch_conv1d_to_rf", "import_params_torch_layer_norm_to_rf"]


def import_params_torch_linear_to_rf(model_pt: torch.nn.Linear, model_rf: Linear):
    """weight transposed, bias as is"""
    if not isinstance(model_pt, torch.nn.Linear) or not isinstance(model_rf, Linear):
        raise TypeError("expected torch.nn.Linear -> rf.Linear, got %s -> %s" % (type(model_pt).__name__, type(model_rf).__name__))
    if model_rf.with_bias != (model_pt.bias is not None):
        raise ValueError("bias on one side only: rf with_bias=%r, torch bias %s" % (model_rf.with_bias, "set" if model_pt.bias is not None else "None"))
    assign(model_rf.weight, model_pt.weight.T, what="Linear.weight")
    if model_rf.with_bias:
        assign(model_rf.bias, model_pt.bias, what="Linear.bias")


def import_params_torch_conv1d_to_rf(model_pt: torch.nn.Conv1d, model_rf: Conv1d):
    """same layout on both sides"""
    if not isinstance(model_pt, torch.nn.Conv1d) or not isinstance(model_rf, Conv1d):
        raise TypeError("expected torch.nn.Conv1d -> rf.Conv1d, got %s -> %s" % (type(model_pt).__name__, type(model_rf).__name__))
    if model_rf.with_bias != (model_pt.bias is not None):
        raise ValueError("bias on one side only: rf with_bias=%r" % model_rf.with_bias)
    assign(model_rf.filter, model_pt.weight, what="Conv1d.filter")
    if model_rf.with_bias:
        assign(model_rf.bias, model_pt.bias, what="Conv1d.bias")


def import_params_torch_layer_norm_to_rf(model_pt: torch.nn.LayerNorm, model_rf: LayerNorm):
    """weight -> scale, bias -> bias"""
    if not isinstance(model_pt, torch.nn.LayerNorm) or not isinstance(model_rf, LayerNorm):
        raise TypeError("expected torch.nn.LayerNorm -> rf.LayerNorm, got %s -> %s" % (type(model_pt).__name__, type(model_rf).__name__))
    assign(model_rf.scale, model_pt.weight, what="LayerNorm.scale")
    assign(model_rf.bias, model_pt.bias, what="LayerNorm.bias")
    check_same_num_params(model_pt, model_rf, what="LayerNorm")
