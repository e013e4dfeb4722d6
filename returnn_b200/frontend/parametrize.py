"""
Parametrization: replace a parameter attribute of a module by a function of that parameter, evaluated at access
(e.g. weight dropout, weight noise).  Parity: returnn/frontend/parametrize.py, parametrizations.py.
"""

from __future__ import annotations
from typing import Optional, Union
from ..tensor import Tensor
from .module import Module
from .parameter import Parameter

__all__ = ["register_parametrization", "remove_parametrization", "is_parametrized", "weight_dropout", "WeightDropout",
           "weight_noise", "WeightNoise"]


def register_parametrization(module: Module, param_name: str, parametrization: Module, *, keep_existing_param: bool = True) -> Module:
    """
    After this, ``module.<param_name>`` evaluates ``parametrization(orig_param)`` on every access.
    The original parameter stays registered under the same checkpoint name when keep_existing_param.
    """
    param = module.__dict__[param_name] if param_name in module.__dict__ else getattr(module, param_name)
    assert isinstance(param, Parameter)
    cls = module.__class__
    if not getattr(cls, "_rf_parametrized", False):
        new_cls = type(cls.__name__, (cls,), {"_rf_parametrized": True, "_rf_orig_cls": cls})
        module.__class__ = new_cls
    store = module.__dict__.setdefault("_rf_parametrizations", {})
    store[param_name] = (param, parametrization)
    del module.__dict__[param_name]
    # keep the Parameter findable for named_parameters under its original name
    module.__dict__["_param_" + param_name] = _ParamHolder(param_name, param, keep_existing_param)

    def getter(self, _n=param_name):
        p, fn = self.__dict__["_rf_parametrizations"][_n]
        return fn(p)

    setattr(module.__class__, param_name, property(getter))
    return module


class _ParamHolder(Module):
    """keeps the raw parameter reachable by module traversal"""

    def __init__(self, name: str, param: Parameter, keep_name: bool):
        super().__init__()
        self.__dict__[name if keep_name else "original"] = param


def _patch_named_parameters():
    orig = Module.named_parameters

    def named_parameters(self, *, recurse: bool = True):
        for name, p in orig(self, recurse=recurse):
            parts = name.split(".")
            parts = [x for x in parts if not x.startswith("_param_")]
            yield ".".join(parts), p

    Module.named_parameters = named_parameters


_patch_named_parameters()


def remove_parametrization(module: Module, param_name: str) -> Module:
    """undo register_parametrization"""
    store = module.__dict__.get("_rf_parametrizations", {})
    param, _ = store.pop(param_name)
    module.__dict__.pop("_param_" + param_name, None)
    delattr(module.__class__, param_name)
    module.__dict__[param_name] = param
    if not store:
        module.__class__ = module.__class__._rf_orig_cls
        module.__dict__.pop("_rf_parametrizations", None)
    return module


def is_parametrized(module: Module, param_name: Optional[str] = None) -> bool:
    """whether a parametrization is registered"""
    store = module.__dict__.get("_rf_parametrizations", {})
    return bool(store) if param_name is None else param_name in store


class WeightDropout(Module):
    """dropout on the weights"""

    def __init__(self, drop_prob: float):
        super().__init__()
        self.drop_prob = drop_prob

    def __call__(self, param: Tensor) -> Tensor:
        from .dropout import dropout
        from .run_ctx import get_run_ctx

        with get_run_ctx().train_flag_ctx(get_run_ctx().is_train_flag_enabled(func=WeightDropout.__call__), func=dropout):
            return dropout(param, self.drop_prob)


def weight_dropout(module: Module, param_name: str, *, drop_prob: float) -> Module:
    """apply WeightDropout to module.param_name"""
    return register_parametrization(module, param_name, WeightDropout(drop_prob))


class WeightNoise(Module):
    """additive Gaussian noise on the weights during training"""

    def __init__(self, std: float):
        super().__init__()
        self.std = std

    def __call__(self, param: Tensor) -> Tensor:
        from .run_ctx import get_run_ctx
        from .rand import random_normal

        flag = get_run_ctx().is_train_flag_enabled(func=WeightNoise.__call__)
        if not (bool(flag.raw_tensor) if isinstance(flag, Tensor) else flag):
            return param
        return param + random_normal(param.dims, dtype=param.dtype, device=param.device, stddev=self.std)


def weight_noise(module: Module, param_name: str, *, std: float) -> Module:
    """apply WeightNoise to module.param_name"""
    return register_parametrization(module, param_name, WeightNoise(std))
