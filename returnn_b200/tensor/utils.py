"""
Helpers to fill tensor templates with seeded random data, incl. random dynamic sizes.
Used by tests and by the dummy datasets.

Parity: returnn/tensor/utils.py:1-243.
"""

from __future__ import annotations
from typing import Optional, Dict, Union, Any
import numpy
from .tensor import Tensor
from .dim import Dim, batch_dim
from .tensor_dict import TensorDict


def tensor_dict_fill_random_numpy_(tensor_dict: TensorDict, *, rnd: Union[int, numpy.random.RandomState] = 42,
                                   dyn_dim_max_sizes: Optional[Dict[Dim, int]] = None,
                                   dyn_dim_min_sizes: Optional[Dict[Dim, int]] = None):
    """fill every template in the dict with random numpy data, as torch tensors"""
    if not isinstance(rnd, numpy.random.RandomState):
        rnd = numpy.random.RandomState(rnd)
    for v in tensor_dict.data.values():
        tensor_fill_random_numpy_(v, rnd=rnd, dyn_dim_max_sizes=dyn_dim_max_sizes, dyn_dim_min_sizes=dyn_dim_min_sizes)


def tensor_fill_random_numpy_(x: Tensor, *, min_val: int = 0, max_val: Optional[int] = None,
                              rnd: numpy.random.RandomState, dyn_dim_max_sizes=None, dyn_dim_min_sizes=None) -> bool:
    """fill x (and sizes of its dynamic dims, if unset) with random data. :return: whether anything was filled"""
    import torch

    filled = False
    dyn_dim_max_sizes = dyn_dim_max_sizes or {}
    dyn_dim_min_sizes = dyn_dim_min_sizes or {}
    for dim in x.dims:
        if dim.is_batch_dim() and dim.dyn_size_ext is None:
            dim.dyn_size_ext = Tensor("batch", dims=[], dtype="int32", raw_tensor=torch.tensor(int(rnd.randint(3, 6)), dtype=torch.int32))
            filled = True
        elif dim.is_dynamic() and (dim.dyn_size_ext is None or dim.dyn_size_ext.raw_tensor is None):
            ext = dim.dyn_size_ext or Tensor("%s:size" % dim.name, dims=[batch_dim], dtype="int32")
            mx = dyn_dim_max_sizes.get(dim, None)
            mn = dyn_dim_min_sizes.get(dim, None)
            if mx is None:
                mx = rnd.randint(5, 20)
            if mn is None:
                mn = max(mx - 5, 1)
            if tensor_fill_random_numpy_(ext, min_val=max(mn, 0), max_val=mx + 1, rnd=rnd):
                # make sure the max is reached so that padding shapes are deterministic
                raw = ext.raw_tensor
                if raw.ndim > 0 and raw.numel() > 0:
                    raw[int(rnd.randint(0, raw.numel()))] = mx
                filled = True
            dim.dyn_size_ext = ext
    if x.raw_tensor is not None:
        return filled
    shape = [d.get_dim_value() for d in x.dims]
    if x.dtype.startswith("int") or x.dtype.startswith("uint"):
        if max_val is None:
            max_val = x.sparse_dim.dimension if x.sparse_dim is not None else rnd.randint(5, 20)
        arr = rnd.randint(min_val, max_val, size=shape, dtype=x.dtype)
    elif x.dtype == "bool":
        arr = rnd.randint(0, 2, size=shape, dtype="int32").astype("bool")
    elif x.dtype.startswith("float") or x.dtype == "bfloat16":
        arr = rnd.normal(0.0, 1.0, size=shape).astype("float32" if x.dtype == "bfloat16" else x.dtype)
    else:
        raise NotImplementedError("fill random: dtype %s" % x.dtype)
    t = torch.from_numpy(numpy.ascontiguousarray(arr))
    if x.dtype == "bfloat16":
        t = t.to(torch.bfloat16)
    x.raw_tensor = t
    return True


def host_to_device(t, device):
    """
    Copy of a host tensor on ``device``. On CUDA it goes through pinned memory and is asynchronous: a plain ``t.to("cuda")`` of a
    pageable tensor synchronises the stream, which drains the queue of kernels the host has issued ahead of the device
    (sequence lengths are moved like this several times per step).
    """
    import torch

    device = torch.device(device)
    if device.type == "cuda" and not t.is_cuda:
        if not t.is_pinned():
            t = t.pin_memory()
        return t.to(device, non_blocking=True)
    return t.to(device)


def tensor_dict_dims_random_seq_len_min_max(tensor_dict, seq_lens=None):
    """
    The dynamic dims of all tensors of the dict (each once, in order of appearance) and the ``(min, max)`` range of lengths to draw for
    each: what :func:`get_random_seq_lens_for_dyn_dims` takes.

    :param seq_lens: a fixed length, a ``(min, max)`` pair, or a dict from data key / Dim / None (default) to either
    :return: dims, {dim: (min, max)}
    Parity: returnn/tensor/utils.py:126.
    """
    if seq_lens is None:
        seq_lens = {}
    if not isinstance(seq_lens, dict):
        seq_lens = {None: seq_lens}

    def as_range(v):
        return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))

    default = as_range(seq_lens.get(None, (2, 11)))
    dims, ranges = [], {}
    for key, t in tensor_dict.data.items():
        for dim in t.dims:
            if dim.is_batch_dim() or dim.is_static() or dim in ranges:
                continue
            dims.append(dim)
            if dim in seq_lens:
                ranges[dim] = as_range(seq_lens[dim])
            elif key in seq_lens:
                ranges[dim] = as_range(seq_lens[key])
            else:
                ranges[dim] = default
    return dims, ranges


def get_random_seq_lens_for_dyn_dims(dims, seq_len_min_max, *, batch_size: int = 1, rnd=1337):
    """
    Random lengths ``[batch_size]`` for every dim, without touching the dims (safe to call from a data thread). The first sequence of every
    dim gets the maximum, so that the padded extent is the same for every seed.

    :return: {dim: int32 array [batch_size]}
    Parity: returnn/tensor/utils.py:194.
    """
    import numpy

    if not isinstance(rnd, numpy.random.RandomState):
        rnd = numpy.random.RandomState(rnd)
    out = {}
    for dim in dims:
        lo, hi = seq_len_min_max[dim]
        lens = rnd.randint(lo, hi + 1, size=[batch_size]).astype("int32")
        if batch_size:
            lens[0] = hi
        out[dim] = lens
    return out
