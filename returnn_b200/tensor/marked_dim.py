"""
Wrappers that mark a :class:`Dim` inside an ``out_shape`` set: implicit dims (a tensor depends on them through a sparse
dim or through dynamic sizes, without having them as an axis) and optional dims.

Parity: returnn/tensor/marked_dim.py:1-83.
"""

from __future__ import annotations
from .dim import Dim


class MarkedDim:
    """base: wraps a Dim"""

    def __init__(self, tag: Dim):
        self.tag = tag

    def __repr__(self):
        return "%s(%r)" % (self.__class__.__name__, self.tag)

    def _eq_tuple(self):
        return self.__class__, self.tag

    def __hash__(self):
        return hash(self._eq_tuple())

    def __eq__(self, other):
        if isinstance(other, MarkedDim):
            return self._eq_tuple() == other._eq_tuple()
        return False

    def __ne__(self, other):
        return not (self == other)

    def __lt__(self, other):
        if not isinstance(other, (Dim, MarkedDim)):
            raise TypeError
        return repr(self) < repr(other)


class ImplicitDim(MarkedDim):
    """a dim the tensor depends on without having it as an axis"""


class ImplicitSparseDim(ImplicitDim):
    """via sparse_dim"""


class ImplicitDynSizeDim(ImplicitDim):
    """via dynamic sizes"""


class OptionalDim(MarkedDim):
    """may or may not be present"""
