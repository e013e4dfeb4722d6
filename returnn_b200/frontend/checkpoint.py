"""
Checkpoints as plain NumPy archives keyed by the RF parameter names, next to the engine's ``.pt`` files: a ``.npz`` written
here can be read without PyTorch and by other tools, and an engine checkpoint converts into it one to one (the state dict of the
engine uses the same names). Plus the bookkeeping that tells which parameters of a model a file covers.

Same functions as returnn/frontend/checkpoint.py:27 (save_params), :45 (load_params), :54 (load_torch_checkpoint),
:74 (check_params_complete); here additionally ``get_model_params`` / ``set_model_params`` for the (eager) module itself.
"""

from __future__ import annotations
from typing import Dict, Optional, Sequence
import numpy
from ..log import log
from .module import Module

__all__ = ["save_params", "load_params", "load_torch_checkpoint", "check_params_complete", "get_model_params", "set_model_params"]

_META_PREFIX = "_"


def save_params(values: Dict[str, numpy.ndarray], filename: str, *, step: Optional[int] = None, epoch: Optional[int] = None):
    """write ``values`` (RF parameter name -> array) to a ``.npz`` file; ``step`` / ``epoch`` travel along as ``_step`` / ``_epoch``"""
    bad = [k for k in values if k.startswith(_META_PREFIX)]
    if bad:
        raise ValueError("parameter names must not start with %r (reserved for meta entries): %s" % (_META_PREFIX, bad))
    meta = {}
    if step is not None:
        meta["_step"] = numpy.array(int(step))
    if epoch is not None:
        meta["_epoch"] = numpy.array(int(epoch))
    numpy.savez(filename, **{k: numpy.asarray(v) for k, v in values.items()}, **meta)
    print("Saved checkpoint %s (%i params)" % (filename, len(values)), file=log.v3)


def load_params(filename: str, *, with_meta: bool = False) -> Dict[str, numpy.ndarray]:
    """the parameters of a file written by :func:`save_params` (without the meta entries unless asked for)"""
    with numpy.load(filename) as data:
        return {name: data[name] for name in data.files if with_meta or not name.startswith(_META_PREFIX)}


def load_torch_checkpoint(filename: str) -> Dict[str, numpy.ndarray]:
    """an engine checkpoint (``{"model": state_dict, "epoch", "step"}`` or a bare state dict) as NumPy arrays by RF parameter name"""
    import torch

    data = torch.load(filename, map_location="cpu", weights_only=False)
    state = data["model"] if isinstance(data, dict) and "model" in data else data
    out = {}
    for name, value in state.items():
        value = value.detach().cpu()
        out[name] = (value.float() if value.dtype == torch.bfloat16 else value).numpy()
    return out


def check_params_complete(model: Module, params: Dict[str, numpy.ndarray], *, allow_missing: bool = False) -> Sequence[str]:
    """
    :return: names of the model parameters that ``params`` provides
    :raise ValueError: a parameter of the model is missing (unless allowed), the file has one the model does not know, or a shape differs
    """
    model_params = dict(model.named_parameters())
    missing = [n for n in model_params if n not in params]
    if missing and not allow_missing:
        raise ValueError("checkpoint is missing: %s" % missing)
    unexpected = [n for n in params if n not in model_params]
    if unexpected:
        raise ValueError("checkpoint has parameters which the model does not: %s" % unexpected)
    for name, p in model_params.items():
        if name in params:
            expected = tuple(d.get_dim_value() for d in p.dims)
            if tuple(params[name].shape) != expected:
                raise ValueError("checkpoint %s has shape %s, model expects %s" % (name, tuple(params[name].shape), expected))
    return [n for n in model_params if n in params]


def get_model_params(model: Module) -> Dict[str, numpy.ndarray]:
    """current values of all parameters (bf16 as float32: NumPy has no bf16)"""
    import torch

    out = {}
    for name, p in model.named_parameters():
        raw = p.raw_tensor.detach().cpu()
        out[name] = (raw.float() if raw.dtype == torch.bfloat16 else raw).numpy().copy()
    return out


def set_model_params(model: Module, params: Dict[str, numpy.ndarray], *, allow_missing: bool = False) -> Sequence[str]:
    """copy ``params`` into the model's parameters (in place, dtype and device of the parameter kept); returns the names that were set"""
    import torch

    names = check_params_complete(model, params, allow_missing=allow_missing)
    model_params = dict(model.named_parameters())
    with torch.no_grad():
        for name in names:
            raw = model_params[name].raw_tensor
            raw.copy_(torch.from_numpy(numpy.ascontiguousarray(params[name])).to(raw.dtype))
    return names
