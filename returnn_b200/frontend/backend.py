"""
Backend selection functions of the frontend API. There is one backend here (PyTorch with the sm_100a kernels) plus the small numpy
backend that ``Tensor`` arithmetic uses for numpy raw tensors; selecting another one raises.  Reference: returnn/frontend/backend.py.
"""

from __future__ import annotations
from .backend_select import select_backend_torch, select_backend_returnn_layers_tf, is_executing_eagerly, get_backend_name

__all__ = ["select_backend", "get_selected_backend", "select_backend_numpy", "select_backend_tf", "select_backend_returnn_layers_tf",
           "select_backend_torch", "is_executing_eagerly", "is_backend_raw_tensor_dim_tag_independent"]


def select_backend(name: str):
    """``"torch"`` (the only full backend) or ``"numpy"``"""
    if name == "torch":
        select_backend_torch()
    elif name == "numpy":
        select_backend_numpy()
    elif name in ("tensorflow", "tf", "returnn_layers_tf"):
        select_backend_tf()
    else:
        raise ValueError("select_backend: unknown backend %r" % (name,))


def get_selected_backend() -> str:
    """name of the selected backend"""
    return get_backend_name()


def select_backend_numpy():
    """numpy raw tensors are handled by the numpy backend whenever they occur; nothing to switch"""


def select_backend_tf():
    """not available: this framework has one backend by design"""
    raise NotImplementedError("the TensorFlow backends are not part of this framework (PyTorch + sm_100a kernels only)")


def is_backend_raw_tensor_dim_tag_independent() -> bool:
    """raw tensors (``torch.Tensor``) know nothing about :class:`Dim`"""
    return True
