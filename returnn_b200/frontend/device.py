"""
Default device handling.  Parity: returnn/frontend/device.py.
"""

from __future__ import annotations
from typing import Optional
import contextlib
from ..tensor import Tensor
from ._utils import wrap

__all__ = ["copy_to_device", "get_default_device", "set_default_device", "set_default_device_ctx", "get_default_dim_size_device"]

_default_device: Optional[str] = None


def copy_to_device(x: Tensor, device: Optional[str] = None) -> Tensor:
    """move to device (default: the default device)"""
    if device is None:
        device = get_default_device()
    if device is None or x.device == str(device):
        return x
    return wrap(x._raw_tensor.to(device), x._dims, like=x)


def get_default_device() -> Optional[str]:
    """device on which new tensors are created"""
    return _default_device


def set_default_device(device: Optional[str]):
    """set it"""
    global _default_device
    _default_device = device


@contextlib.contextmanager
def set_default_device_ctx(device: Optional[str]):
    """temporarily set it"""
    global _default_device
    old = _default_device
    _default_device = device
    try:
        yield
    finally:
        _default_device = old


def get_default_dim_size_device() -> Optional[str]:
    """where the size tensors of dynamic dims (``Dim.dyn_size_ext``) live: on the host, so that shapes are known without a device read"""
    return "cpu"
