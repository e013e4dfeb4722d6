"""
``extern_data``: the typed description of a batch and its conversion from the raw collated dict to a
:class:`TensorDict` on the device. Sequence lengths stay on the host.

Parity: returnn/torch/data/extern_data.py (extern_data_template_from_config_opts :13-24,
raw_dict_to_extern_data :27-104, split/can-split batch for OOM retry :107-277).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union
import numpy
import torch
from ...tensor import Tensor, TensorDict, Dim, batch_dim
from ...frontend._utils import dtype_name, torch_dtype


def extern_data_template_from_config_opts(extern_data_dict: Dict[str, Any]) -> TensorDict:
    """config ``extern_data`` -> TensorDict of templates"""
    extern_data = TensorDict()
    extern_data.update(extern_data_dict, auto_convert=True)
    if "seq_tag" not in extern_data.data:
        extern_data.data["seq_tag"] = Tensor("seq_tag", dims=[batch_dim], dtype="string")
    return extern_data


def raw_dict_to_extern_data(extern_data_raw: Dict[str, Any], *, extern_data_template: TensorDict,
                            device: Union[str, torch.device], float_dtype: Optional[Union[str, torch.dtype]] = None,
                            with_eval_targets: bool = False, non_blocking: bool = True) -> TensorDict:
    """
    :param extern_data_raw: output of collate_batch
    :param with_eval_targets: also take keys with available_for_inference=False
    :return: filled copy of the template; dynamic dims get their sizes (host tensors), batch_dim its size
    """
    if isinstance(float_dtype, torch.dtype):
        float_dtype = dtype_name(float_dtype)
    extern_data = TensorDict()
    batch_size_set = False
    for k, data in extern_data_template.data.items():
        data = data.copy_template()
        if not with_eval_targets and not data.available_for_inference:
            continue
        if k not in extern_data_raw:
            if k == "seq_tag":
                continue
            raise KeyError("extern_data key %r missing in the batch; have %r" % (k, sorted(extern_data_raw.keys())))
        raw = extern_data_raw[k]
        if data.dtype == "string":
            t = Tensor.__new__(Tensor)
            for slot in Tensor.__slots__:
                object.__setattr__(t, slot, getattr(data, slot, None))
            t._raw_tensor = raw
            extern_data.data[k] = t
            continue
        assert isinstance(raw, torch.Tensor), "extern_data %r: expected torch.Tensor, got %r" % (k, type(raw))
        if extern_data_raw.get("%s:packed" % k):
            raise ValueError("extern_data %r is packed; use packed_tensors handling (rf.pack_import)" % k)
        # copy first (asynchronous from pinned memory), convert on the device: a conversion on the host would leave
        # pinned memory and make the copy a synchronising one
        if str(raw.device) != str(device):
            raw = raw.to(device, non_blocking=non_blocking)
        if data.dtype != dtype_name(raw.dtype):
            raw = raw.to(torch_dtype(data.dtype))
        if float_dtype and raw.is_floating_point() and dtype_name(raw.dtype) != float_dtype:
            raw = raw.to(torch_dtype(float_dtype))
            data.dtype = float_dtype
        assert raw.ndim == len(data.dims), "extern_data %r: batch has ndim %i, template %r" % (k, raw.ndim, data)
        if not batch_size_set and data.dims and data.dims[0].is_batch_dim():
            batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(raw.shape[0], dtype=torch.int32))
            batch_size_set = True
        # dynamic sizes: first dynamic non-batch dim gets "<key>:seq_len"
        seq_len_key = "%s:seq_len" % k
        first_dyn = True
        for i, dim in enumerate(data.dims):
            if dim.is_batch_dim() or dim.is_static():
                if dim.is_static():
                    assert dim.dimension == raw.shape[i], "extern_data %r: shape %r does not match %r" % (k, tuple(raw.shape), data)
                continue
            if first_dyn and seq_len_key in extern_data_raw:
                sizes = extern_data_raw[seq_len_key]
                assert isinstance(sizes, torch.Tensor) and sizes.ndim == 1
                if dim.dyn_size_ext is None or dim.dyn_size_ext.raw_tensor is not sizes:
                    dim.dyn_size_ext = Tensor("%s:seq_len" % k, dims=[batch_dim], dtype=dtype_name(sizes.dtype), raw_tensor=sizes)
            else:
                dim.dyn_size_ext = Tensor("%s:size%i" % (k, i), dims=[], dtype="int32", raw_tensor=torch.tensor(raw.shape[i], dtype=torch.int32))
            first_dyn = False
        if str(raw.device) != str(device):
            raw = raw.to(device, non_blocking=non_blocking)
        data._raw_tensor = raw
        extern_data.data[k] = data
    return extern_data


def raw_dict_can_split_batch(extern_data_raw: Dict[str, Any]) -> bool:
    """more than one sequence in the batch"""
    for v in extern_data_raw.values():
        if isinstance(v, (torch.Tensor, numpy.ndarray)) and v.ndim >= 1:
            return v.shape[0] > 1
    return False


def raw_dict_split_batch(extern_data_raw: Dict[str, Any], *, splits: Union[int, Sequence[int]] = 2) -> List[Dict[str, Any]]:
    """split along the batch axis into parts (for OOM retry); padding is cut to each part's longest sequence"""
    some = next(v for v in extern_data_raw.values() if isinstance(v, (torch.Tensor, numpy.ndarray)) and v.ndim >= 1)
    n = some.shape[0]
    if isinstance(splits, int):
        base, extra = divmod(n, splits)
        splits = [base + (1 if i < extra else 0) for i in range(splits)]
    splits = [s for s in splits if s > 0]
    assert sum(splits) == n
    res = []
    offset = 0
    for s in splits:
        part: Dict[str, Any] = {}
        for k, v in extern_data_raw.items():
            if isinstance(v, (torch.Tensor, numpy.ndarray)) and v.ndim >= 1 and v.shape[0] == n:
                part[k] = v[offset: offset + s]
            else:
                part[k] = v
        for k in list(part.keys()):
            if k.endswith(":seq_len"):
                key = k[: -len(":seq_len")]
                if key in part and isinstance(part[key], torch.Tensor) and part[key].ndim >= 2:
                    mx = int(part[k].max()) if part[k].numel() else 0
                    part[key] = part[key][:, :mx]
        res.append(part)
        offset += s
    return res


def get_batch_dim_from_extern_data(extern_data: TensorDict) -> Dim:
    """
    The batch dim of a collated batch: by construction the first dim of every tensor (``collate_batch``). It need not be the global
    ``batch_dim`` object and need not even be marked as a batch dim. Parity: returnn/torch/data/extern_data.py:292.
    """
    return next(iter(extern_data.data.values())).dims[0]
