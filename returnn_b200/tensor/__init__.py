"""
Named-dimension tensors: :class:`Tensor`, :class:`Dim`, :class:`TensorDict`.
"""

from .dim import Dim, batch_dim, single_step_dim, DimTypes, VerifyOutShapeException
from .tensor import Tensor
from .tensor_dict import TensorDict
from .marked_dim import MarkedDim, ImplicitDim, ImplicitSparseDim, ImplicitDynSizeDim, OptionalDim
from .control_flow_ctx import ControlFlowContext

__all__ = [
    "Tensor",
    "Dim",
    "TensorDict",
    "batch_dim",
    "single_step_dim",
    "DimTypes",
    "VerifyOutShapeException",
    "MarkedDim",
    "ImplicitDim",
    "ImplicitSparseDim",
    "ImplicitDynSizeDim",
    "OptionalDim",
    "ControlFlowContext",
]
