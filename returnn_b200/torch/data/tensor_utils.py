"""In-place conversion of the raw tensors of ``Tensor`` / ``TensorDict`` between numpy and torch (dynamic sizes included). Parity: returnn/torch/data/tensor_utils.py."""

from __future__ import annotations
import numpy
import torch
from ...tensor import Tensor, TensorDict


def tensor_numpy_to_torch_(x: Tensor):
    """numpy raw tensor (and those of the dims' dynamic sizes) -> torch, in place; strings and objects stay numpy"""
    if x.raw_tensor is None or isinstance(x.raw_tensor, torch.Tensor):
        pass
    elif isinstance(x.raw_tensor, numpy.ndarray) and x.raw_tensor.dtype.kind not in "OUS":
        x._raw_tensor = torch.from_numpy(numpy.ascontiguousarray(x.raw_tensor))
    for dim in x.dims:
        ext = dim.dyn_size_ext
        if ext is not None and isinstance(ext.raw_tensor, numpy.ndarray):
            ext._raw_tensor = torch.from_numpy(numpy.ascontiguousarray(ext.raw_tensor))


def tensor_dict_numpy_to_torch_(x: TensorDict):
    """every tensor of the dict, in place"""
    for v in x.data.values():
        tensor_numpy_to_torch_(v)


def tensor_torch_to_numpy_(x: Tensor):
    """torch raw tensor (and those of the dims' dynamic sizes) -> numpy on the host, in place"""
    if isinstance(x.raw_tensor, torch.Tensor):
        t = x.raw_tensor.detach().cpu()
        x._raw_tensor = (t.float() if t.dtype == torch.bfloat16 else t).numpy()
    for dim in x.dims:
        ext = dim.dyn_size_ext
        if ext is not None and isinstance(ext.raw_tensor, torch.Tensor):
            ext._raw_tensor = ext.raw_tensor.detach().cpu().numpy()


def tensor_dict_torch_to_numpy_(x: TensorDict):
    """every tensor of the dict, in place"""
    for v in x.data.values():
        tensor_torch_to_numpy_(v)
