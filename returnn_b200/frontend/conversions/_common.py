"""helpers shared by the importers"""

from __future__ import annotations
from typing import Iterable
import torch


def num_params_torch(module: torch.nn.Module) -> int:
    """element count over ``named_parameters`` of a torch module"""
    return sum(p.numel() for _, p in module.named_parameters())


def num_params_rf(module) -> int:
    """element count over the parameters of an RF module"""
    return sum(p.num_elements() for _, p in module.named_parameters())


def check_same_num_params(src: torch.nn.Module, dst, *, what: str, exclude_rf: Iterable = ()):
    """an import that covered every tensor leaves no parameter on either side unaccounted for"""
    n_src = num_params_torch(src)
    n_dst = num_params_rf(dst) - sum(p.num_elements() for p in exclude_rf)
    if n_src != n_dst:
        raise ValueError("%s: the source has %i parameter elements, the RF module %i" % (what, n_src, n_dst))


def assign(param, value: torch.Tensor, *, what: str):
    """``param.raw_tensor[...] = value`` with a shape check that names the parameter"""
    raw = param.raw_tensor
    if tuple(raw.shape) != tuple(value.shape):
        raise ValueError("%s: shape %s in the RF module, %s in the source" % (what, tuple(raw.shape), tuple(value.shape)))
    with torch.no_grad():
        raw.copy_(value.to(raw.dtype))
