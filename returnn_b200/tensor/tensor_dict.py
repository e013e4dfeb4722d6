"""
``TensorDict``: ordered mapping name -> :class:`Tensor`, with conversion from config templates
(``extern_data`` / ``model_outputs``) and to/from flat raw dicts (``"<key>:size<axis>"`` entries for dynamic sizes).

Parity: returnn/tensor/tensor_dict.py:1-190.
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Sequence, Union
from .tensor import Tensor
from .dim import Dim, batch_dim


def _tensor_from_template_dict(name: str, opts: Dict[str, Any]) -> Tensor:
    opts = dict(opts)
    if "dim_tags" in opts:
        opts["dims"] = opts.pop("dim_tags")
    if "dims" not in opts:
        # legacy {"dim": F, "shape": (None, F), "sparse": bool}
        shape = opts.pop("shape", None)
        dim = opts.pop("dim", None)
        sparse = opts.pop("sparse", False)
        if shape is None:
            shape = (None,) if sparse else (None, dim)
        dims = [batch_dim]
        for i, s in enumerate(shape):
            if s is None:
                dims.append(Dim(None, name="%s:time%i" % (name, i) if i else "%s:time" % name, kind=Dim.Types.Spatial))
            else:
                dims.append(Dim(int(s), name="%s:feature" % name, kind=Dim.Types.Feature))
        opts["dims"] = dims
        if sparse:
            opts["sparse_dim"] = Dim(int(dim), name="%s:classes" % name, kind=Dim.Types.Feature)
            opts.setdefault("dtype", "int32")
    opts.pop("vocab", None)
    opts.pop("time_dim_axis", None)
    return Tensor(name=name, **opts)


class TensorDict:
    """name -> Tensor"""

    def __init__(self, data: Optional[Union[Dict[str, Union[Tensor, Dict[str, Any]]], "TensorDict", Sequence[Tensor]]] = None):
        self.data: Dict[str, Tensor] = {}
        if data is not None:
            self.update(data)

    def __repr__(self):
        return "TensorDict(%r)" % (self.data,)

    def update(self, data, *, auto_convert: bool = False):
        """merge"""
        if isinstance(data, TensorDict):
            for k, v in data.data.items():
                self.data[k] = v.copy()
        elif isinstance(data, dict):
            for k, v in data.items():
                if isinstance(v, dict):
                    v = _tensor_from_template_dict(k, v)
                elif auto_convert and not isinstance(v, Tensor):
                    raise TypeError("TensorDict: cannot convert %r" % (v,))
                assert isinstance(v, Tensor), "TensorDict: %r: expected Tensor, got %r" % (k, type(v))
                self.data[k] = v
        elif isinstance(data, (list, tuple)):
            for v in data:
                assert isinstance(v, Tensor)
                self.data[v.name] = v
        else:
            raise TypeError("invalid data %r" % type(data))

    def __getitem__(self, item: str) -> Tensor:
        return self.data[item]

    def __setitem__(self, key: str, value: Tensor):
        self.data[key] = value

    def __contains__(self, item):
        return item in self.data

    def __iter__(self):
        return iter(self.data)

    def __len__(self):
        return len(self.data)

    def get(self, key, default=None):
        """dict.get"""
        return self.data.get(key, default)

    def keys(self):
        """keys"""
        return self.data.keys()

    def values(self):
        """values"""
        return self.data.values()

    def items(self):
        """items"""
        return self.data.items()

    def reset_content(self):
        """drop raw tensors and dynamic sizes"""
        for v in self.data.values():
            v._raw_tensor = None
            for d in v.dims:
                if d.is_dynamic():
                    d.reset_raw()

    def copy_template(self) -> "TensorDict":
        """templates only"""
        return TensorDict({k: v.copy_template() for k, v in self.data.items()})

    def as_raw_tensor_dict(self, *, include_const_sizes: bool = False, include_scalar_dyn_sizes: bool = True,
                           exclude_duplicate_dims: bool = False, expected_value_type=object) -> Dict[str, Any]:
        """flat dict: key -> raw, "key:size<i>" -> raw sizes of dynamic axis i"""
        out: Dict[str, Any] = {}
        visited = set()
        for key, value in self.data.items():
            assert key not in out
            assert value.raw_tensor is not None, "TensorDict.as_raw_tensor_dict: %r has no raw tensor" % value
            out[key] = value.raw_tensor
            for i, dim in enumerate(value.dims):
                if exclude_duplicate_dims and dim in visited:
                    continue
                visited.add(dim)
                k = "%s:size%i" % (key, i)
                if dim.is_batch_dim() and (dim.dyn_size_ext is None or dim.dyn_size_ext.raw_tensor is None):
                    if include_scalar_dyn_sizes:
                        import torch

                        out[k] = torch.tensor(value.raw_tensor.shape[i], dtype=torch.int32)
                elif dim.is_dynamic():
                    ext = dim.dyn_size_ext
                    if ext is None or ext.raw_tensor is None:
                        continue
                    if not include_scalar_dyn_sizes and not ext.dims:
                        continue
                    out[k] = ext.raw_tensor
                elif include_const_sizes:
                    out[k] = dim.dimension
        return out

    def assign_from_raw_tensor_dict_(self, raw_tensor_dict: Dict[str, Any], *, with_scalar_dyn_sizes: bool = True,
                                     duplicate_dims_are_excluded: bool = False):
        """inverse of as_raw_tensor_dict"""
        from .tensor import _raw_dtype_str

        visited = set()
        for key, value in self.data.items():
            raw = raw_tensor_dict[key]
            for i, dim in enumerate(value.dims):
                k = "%s:size%i" % (key, i)
                if duplicate_dims_are_excluded and dim in visited:
                    continue
                visited.add(dim)
                if dim.is_dynamic() and k in raw_tensor_dict:
                    sizes = raw_tensor_dict[k]
                    ndim = getattr(sizes, "ndim", 0)
                    if dim.is_batch_dim() and ndim == 0:
                        dim.dyn_size_ext = Tensor("batch:size", dims=[], dtype=_raw_dtype_str(sizes), raw_tensor=sizes)
                    elif ndim == 0:
                        if with_scalar_dyn_sizes:
                            dim.dyn_size_ext = Tensor("%s:size" % dim.name, dims=[], dtype=_raw_dtype_str(sizes), raw_tensor=sizes)
                    else:
                        dim.dyn_size_ext = Tensor("%s:size" % dim.name, dims=[batch_dim], dtype=_raw_dtype_str(sizes), raw_tensor=sizes)
            value.raw_tensor = raw
