"""
``Linear`` and ``Embedding``.  Weight layout is ``[in, out]`` (in-major) as in the checkpoint format.

Parity: returnn/frontend/linear.py:14-58.
"""

from __future__ import annotations
from typing import Optional
import torch
from ..tensor import Tensor, Dim
from .module import Module
from .parameter import Parameter
from . import init as _init
from ._utils import wrap

__all__ = ["Linear", "Embedding"]


class Linear(Module):
    """``y = x @ weight + bias`` over in_dim"""

    def __init__(self, in_dim: Dim, out_dim: Dim, *, with_bias: bool = True):
        super().__init__()
        assert isinstance(in_dim, Dim) and isinstance(out_dim, Dim)
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.weight = Parameter((in_dim, out_dim))
        self.weight.initial = _init.Glorot()
        self.with_bias = with_bias
        self.bias = None
        if with_bias:
            self.bias = Parameter((out_dim,))
            self.bias.initial = 0.0

    def __call__(self, source: Tensor) -> Tensor:
        if not isinstance(source, Tensor):
            raise TypeError("%s: source must be a Tensor, got %r" % (self, type(source)))
        dims = source._dims
        if self.in_dim not in dims:
            raise ValueError("%s: input %r does not have in_dim %r" % (self, source, self.in_dim))
        raw = source._raw_tensor
        if dims[-1] != self.in_dim:
            from ._utils import axis_of

            ax = axis_of(source, self.in_dim)
            raw = raw.movedim(ax, -1)
            dims = tuple(d for d in dims if d != self.in_dim) + (self.in_dim,)
        from ..ops import linear as _lin

        w = self.weight
        w_raw = w._raw_tensor
        if w.dims[0] != self.in_dim and w.dims[0] == self.out_dim and w.dims[-1] == self.in_dim:
            # a weight stored [out, in]: e.g. output logits tied to the [vocab, model] table of an Embedding
            w_raw = w_raw.t()
        out = _lin.linear(raw, w_raw, self.bias._raw_tensor if self.bias is not None else None)
        return wrap(out, dims[:-1] + (self.out_dim,), feature_dim=self.out_dim)


class Embedding(Module):
    """lookup of class indices in a ``[vocab, out]`` table"""

    def __init__(self, in_dim: Dim, out_dim: Dim):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.weight = Parameter((in_dim, out_dim))
        self.weight.initial = _init.Glorot()

    def __call__(self, source: Tensor) -> Tensor:
        if not isinstance(source, Tensor):
            raise TypeError("%s: source must be a Tensor, got %r" % (self, type(source)))
        if source.sparse_dim != self.in_dim and source.sparse_dim is not None:
            raise ValueError("%s: input %r sparse dim does not match %r" % (self, source, self.in_dim))
        idx = source._raw_tensor
        out = torch.nn.functional.embedding(idx if idx.dtype in (torch.int32, torch.int64) else idx.long(), self.weight._raw_tensor)
        return wrap(out, source._dims + (self.out_dim,), feature_dim=self.out_dim)
