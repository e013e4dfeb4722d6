"""
``Parameter``: a :class:`Tensor` whose raw tensor is a ``torch.nn.Parameter`` (or a plain buffer when ``auxiliary``).

Parity: returnn/frontend/parameter.py:19 (initial, trainable, auxiliary, weight_decay, non_critical_for_restore).
"""

from __future__ import annotations
from typing import Optional, Sequence, Union, Callable
import numpy
import torch
from ..tensor import Tensor, Dim
from ._utils import torch_dtype, get_default_float_dtype, dtype_name

__all__ = ["Parameter", "set_parameter_copy_behavior_ctx"]


class Parameter(Tensor):
    """
    Model parameter. All dims must be static.
    """

    __slots__ = ("_trainable", "_auxiliary", "_initial", "weight_decay", "non_critical_for_restore", "__dict__")

    def __init__(self, dims: Sequence[Dim], dtype: Optional[str] = None, *, sparse_dim: Optional[Dim] = None,
                 trainable: Optional[bool] = None, auxiliary: bool = False, non_critical_for_restore: bool = False,
                 weight_decay: Optional[float] = 0.0, initial=None, raw_tensor=None, device: Optional[str] = None):
        """
        :param trainable: default: float params which are not auxiliary
        :param auxiliary: not updated by the optimizer (e.g. running statistics); becomes a buffer in the state dict
        :param non_critical_for_restore: may be missing in a checkpoint
        :param weight_decay: relative weight decay factor for this param (0 disables)
        :param initial: value or ParamInit callable
        """
        dims = tuple(dims)
        for d in dims:
            assert isinstance(d, Dim) and d.is_static(), "Parameter: dims must be static, got %r" % (d,)
        if dtype is None:
            dtype = "int32" if sparse_dim is not None else get_default_float_dtype()
        super().__init__("parameter", dims=dims, dtype=dtype, sparse_dim=sparse_dim)
        if trainable is None:
            trainable = (not auxiliary) and (dtype.startswith("float") or dtype == "bfloat16")
        if raw_tensor is None:
            if device is None:
                from .device import get_default_device

                device = get_default_device()
            data = torch.zeros([d.dimension for d in dims], dtype=torch_dtype(dtype), device=device)
            raw_tensor = torch.nn.Parameter(data, requires_grad=bool(trainable))
        self._raw_tensor = raw_tensor
        self._trainable = bool(trainable)
        self._auxiliary = auxiliary
        self._initial = None
        self.weight_decay = weight_decay
        self.non_critical_for_restore = non_critical_for_restore
        if initial is not None:
            self.initial = initial

    def __copy__(self):
        if _copy_behavior == "share":
            return self
        res = type(self)(dims=self.dims, dtype=self.dtype, trainable=self.trainable, auxiliary=self.auxiliary,
                         non_critical_for_restore=self.non_critical_for_restore, weight_decay=self.weight_decay)
        res.name = self.name
        res._initial = self._initial
        with torch.no_grad():
            res._raw_tensor.copy_(self._raw_tensor)
        return res

    def __deepcopy__(self, memo=None):
        return self.__copy__()

    @property
    def initial(self):
        """initial value or initializer"""
        return self._initial

    @initial.setter
    def initial(self, value):
        from .init import ParamInit

        self._initial = value
        if isinstance(value, ParamInit) or (callable(value) and not isinstance(value, Tensor)):
            value = value(dims=self.dims, dtype=self.dtype, sparse_dim=self.sparse_dim, device=self.device)
        self.assign(value)

    def assign(self, value):
        """overwrite the value in place"""
        with torch.no_grad():
            raw = self._raw_tensor
            if isinstance(value, Tensor):
                raw.copy_(value.copy_compatible_to_dims_raw(self.dims))
            elif isinstance(value, (torch.Tensor, numpy.ndarray)):
                raw.copy_(torch.as_tensor(value))
            elif value is None:
                raw.zero_()
            else:
                raw.fill_(value)

    def assign_add(self, value):
        """+= in place"""
        with torch.no_grad():
            self._raw_tensor.add_(value.copy_compatible_to_dims_raw(self.dims) if isinstance(value, Tensor) else value)

    def assign_key(self, axis, key, value, key_dim=None):
        """self[key along axis] = value"""
        from ._utils import axis_of

        with torch.no_grad():
            ax = axis_of(self, axis)
            idx = [slice(None)] * self._raw_tensor.ndim
            idx[ax] = key._raw_tensor.long() if isinstance(key, Tensor) else key
            self._raw_tensor[tuple(idx)] = value._raw_tensor if isinstance(value, Tensor) else value

    @property
    def trainable(self) -> bool:
        """updated by the optimizer"""
        return self._trainable

    @trainable.setter
    def trainable(self, value: bool):
        self._trainable = bool(value)
        if isinstance(self._raw_tensor, torch.nn.Parameter):
            self._raw_tensor.requires_grad_(bool(value))

    @property
    def auxiliary(self) -> bool:
        """not a learned weight"""
        return self._auxiliary

    @auxiliary.setter
    def auxiliary(self, value: bool):
        self._auxiliary = value

    def __repr__(self):
        return "Parameter{%r, [%s], %s}" % (self.name, ",".join(d.short_repr() for d in self.dims), self.dtype)


_copy_behavior = "copy_init"


import contextlib as _contextlib


@_contextlib.contextmanager
def set_parameter_copy_behavior_ctx(mode: str):
    """
    What ``copy.copy`` / ``copy.deepcopy`` of a parameter gives inside the block: ``"copy_init"`` (default) a new parameter of its
    own, ``"share"`` the very same parameter (deep copies of a module then share their weights with the original).
    Reference: returnn/frontend/parameter.py:262-282.
    """
    global _copy_behavior
    assert mode in ("copy_init", "share")
    old = _copy_behavior
    try:
        _copy_behavior = mode
        yield
    finally:
        _copy_behavior = old
