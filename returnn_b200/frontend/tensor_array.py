"""
``TensorArray``: growable list of same-shaped tensors that can be stacked along a new dim (used by ``rf.scan``).
Parity: returnn/frontend/tensor_array.py.
"""

from __future__ import annotations
from typing import List, Optional, Sequence, Tuple
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap

__all__ = ["TensorArray"]


class TensorArray:
    """list of tensors"""

    def __init__(self, tensor_template: Tensor, *, _items: Optional[List[Tensor]] = None):
        self.tensor_template = tensor_template
        self._items: List[Tensor] = list(_items) if _items else []

    @classmethod
    def unstack(cls, tensor: Tensor, *, axis: Dim) -> "TensorArray":
        """split along axis"""
        from ._utils import axis_of

        ax = axis_of(tensor, axis)
        dims = [d for d in tensor.dims if d != axis]
        items = [wrap(r, dims, like=tensor) for r in torch.unbind(tensor.raw_tensor, dim=ax)]
        return cls(items[0].copy_template() if items else tensor.copy_template_excluding_axis(ax), _items=items)

    def __len__(self):
        return len(self._items)

    def __getitem__(self, index) -> Tensor:
        if isinstance(index, Tensor):
            index = int(index.raw_tensor)
        return self._items[index]

    def push_back(self, tensor: Tensor) -> "TensorArray":
        """append; returns self"""
        self._items.append(tensor)
        return self

    def stack(self, *, axis: Dim) -> Tensor:
        """stack along a new first axis"""
        if not self._items:
            dims = [axis] + list(self.tensor_template.dims)
            from ._utils import torch_dtype

            shape = [0] + [d.get_dim_value() for d in self.tensor_template.dims]
            return wrap(torch.zeros(shape, dtype=torch_dtype(self.tensor_template.dtype)), dims)
        dims0 = self._items[0].dims
        raws = [t.copy_compatible_to_dims_raw(dims0) for t in self._items]
        # items may differ in broadcastable sizes (e.g. growing dims are not supported here)
        raw = torch.stack(raws, dim=0)
        if axis.is_dynamic() and (axis.dyn_size_ext is None or axis.dyn_size_ext.raw_tensor is None):
            axis.dyn_size_ext = Tensor("%s:size" % axis.name, dims=[], dtype="int32", raw_tensor=torch.tensor(len(raws), dtype=torch.int32))
        return wrap(raw, [axis] + list(dims0), like=self._items[0])
