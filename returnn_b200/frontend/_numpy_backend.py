"""
Minimal NumPy backend: compare / combine / reduce / where / range / activations on :class:`Tensor` objects whose raw tensor
is a ``numpy.ndarray``. Used on the dataset side (post-processing functions that do a little named-dim math on a
sequence) and in tests, where no device and no autograd is wanted. The functions of :mod:`returnn_b200.frontend` dispatch
here when they see NumPy raw tensors.

Parity: returnn/frontend/_numpy_backend.py (NumpyBackend :18-267).
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union
import numpy
from ..tensor import Tensor, Dim

_CMP = {
    "==": numpy.equal, "equal": numpy.equal, "!=": numpy.not_equal, "not_equal": numpy.not_equal, "<": numpy.less, "less": numpy.less,
    "<=": numpy.less_equal, "less_equal": numpy.less_equal, ">": numpy.greater, "greater": numpy.greater, ">=": numpy.greater_equal,
    "greater_equal": numpy.greater_equal,
}
_BIN = {
    "+": numpy.add, "add": numpy.add, "-": numpy.subtract, "sub": numpy.subtract, "*": numpy.multiply, "mul": numpy.multiply,
    "/": numpy.true_divide, "truediv": numpy.true_divide, "//": numpy.floor_divide, "floordiv": numpy.floor_divide, "%": numpy.mod, "mod": numpy.mod,
    "**": numpy.power, "pow": numpy.power, "max": numpy.maximum, "maximum": numpy.maximum, "min": numpy.minimum, "minimum": numpy.minimum,
    "logical_and": numpy.logical_and, "logical_or": numpy.logical_or, "squared_difference": lambda a, b: numpy.square(a - b),
}
_ACT = {
    "exp": numpy.exp, "log": numpy.log, "sqrt": numpy.sqrt, "abs": numpy.abs, "neg": numpy.negative, "tanh": numpy.tanh, "sin": numpy.sin,
    "cos": numpy.cos, "ceil": numpy.ceil, "floor": numpy.floor, "round": numpy.round, "square": numpy.square, "logical_not": numpy.logical_not,
    "sigmoid": lambda x: 1.0 / (1.0 + numpy.exp(-x)), "relu": lambda x: numpy.maximum(x, 0), "rsqrt": lambda x: 1.0 / numpy.sqrt(x),
    "reciprocal": lambda x: 1.0 / x, "log1p": numpy.log1p, "expm1": numpy.expm1,
}


def is_numpy(x) -> bool:
    """a Tensor with a NumPy raw tensor, or a raw NumPy array"""
    if isinstance(x, Tensor):
        x = x._raw_tensor
    return isinstance(x, (numpy.ndarray, numpy.generic))


class NumpyBackend:
    """static functions, named like the backend interface of the reference"""

    name = "numpy"
    RawTensorType = numpy.ndarray

    @staticmethod
    def executing_eagerly() -> bool:
        """always"""
        return True

    @staticmethod
    def assert_(condition: Tensor, message: str, *, stop: bool = True):
        """host check"""
        if not bool(numpy.all(condition.raw_tensor)):
            if stop:
                raise AssertionError(message)
            print("[ASSERT FAILED WARNING]: %s" % message)

    @staticmethod
    def get_dtype_name_raw(raw_tensor: numpy.ndarray) -> str:
        """e.g. "float32"; strings and objects map to "string" / "object" """
        kind = raw_tensor.dtype.kind
        if kind in "US":
            return "string"
        if kind == "O":
            return "object"
        return raw_tensor.dtype.name

    @staticmethod
    def as_dtype_raw(dtype_name: str) -> numpy.dtype:
        """name -> numpy dtype"""
        return numpy.dtype(object if dtype_name in ("string", "object") else dtype_name)

    @staticmethod
    def get_ndim_raw(raw_tensor: numpy.ndarray) -> int:
        """number of axes"""
        return raw_tensor.ndim

    @staticmethod
    def get_shape_raw(raw_tensor: numpy.ndarray) -> Tuple[int, ...]:
        """shape"""
        return tuple(raw_tensor.shape)

    get_shape_tuple_raw = get_shape_raw
    get_known_shape_raw = get_shape_raw

    @staticmethod
    def convert_to_tensor(value, *, dims: Sequence[Dim] = (), dtype: Optional[str] = None, sparse_dim: Optional[Dim] = None, name: Optional[str] = None) -> Tensor:
        """Python / NumPy value -> Tensor with a NumPy raw tensor"""
        if isinstance(value, Tensor):
            return value
        arr = numpy.asarray(value, dtype=dtype) if dtype else numpy.asarray(value)
        if arr.dtype == numpy.float64 and dtype is None and not isinstance(value, numpy.ndarray):
            arr = arr.astype("float32")
        if arr.dtype == numpy.int64 and dtype is None and not isinstance(value, numpy.ndarray):
            arr = arr.astype("int32")
        assert arr.ndim == len(dims), "convert_to_tensor: value has %i axes, dims %r" % (arr.ndim, dims)
        return Tensor(name or "const", dims=list(dims), dtype=NumpyBackend.get_dtype_name_raw(arr), sparse_dim=sparse_dim, raw_tensor=arr)

    @staticmethod
    def expand_dims_raw(raw_tensor: numpy.ndarray, axis: int) -> numpy.ndarray:
        """new axis of size 1"""
        return numpy.expand_dims(raw_tensor, axis)

    @staticmethod
    def transpose_raw(raw_tensor: numpy.ndarray, perm: Sequence[int]) -> numpy.ndarray:
        """permute axes"""
        return numpy.transpose(raw_tensor, list(perm))

    @staticmethod
    def reshape_raw(raw_tensor: numpy.ndarray, shape: Sequence[int]) -> numpy.ndarray:
        """reshape"""
        return numpy.reshape(raw_tensor, tuple(shape))

    @staticmethod
    def compare_raw(a: numpy.ndarray, kind: str, b: numpy.ndarray) -> numpy.ndarray:
        """elementwise comparison"""
        return _CMP[kind](a, b)

    @staticmethod
    def combine_raw(a: numpy.ndarray, kind: str, b: numpy.ndarray) -> numpy.ndarray:
        """elementwise binary op"""
        return _BIN[kind](a, b)

    @staticmethod
    def activation_raw(raw_tensor: numpy.ndarray, func: str) -> numpy.ndarray:
        """elementwise unary op by name"""
        return _ACT[func](raw_tensor)

    # -- named-dim level -------------------------------------------------------------------------------------------
    @staticmethod
    def _to_dims(x: Tensor, out_dims: Sequence[Dim]) -> numpy.ndarray:
        """raw tensor of x broadcast-compatible to out_dims (missing dims become size-1 axes, order as out_dims)"""
        raw = numpy.asarray(x._raw_tensor)
        have = list(x._dims)
        perm = [have.index(d) for d in out_dims if d in have]
        raw = numpy.transpose(raw, perm) if perm != list(range(len(perm))) else raw
        shape = []
        it = iter(raw.shape)
        for d in out_dims:
            shape.append(next(it) if d in have else 1)
        return raw.reshape(shape)

    @staticmethod
    def _merge_dims(a: Tensor, b: Tensor) -> Tuple[Dim, ...]:
        out = list(a._dims)
        for d in b._dims:
            if d not in out:
                out.append(d)
        if len(b._dims) > len(a._dims) and set(a._dims) <= set(b._dims):
            out = list(b._dims)
        return tuple(out)

    @staticmethod
    def _binary(a, kind: str, b, table) -> Tensor:
        if not isinstance(a, Tensor):
            a = NumpyBackend.convert_to_tensor(a, dtype=b.dtype if isinstance(b, Tensor) and not isinstance(a, (bool, numpy.bool_)) else None)
        if not isinstance(b, Tensor):
            b = NumpyBackend.convert_to_tensor(b, dtype=a.dtype if not isinstance(b, (bool, numpy.bool_)) else None)
        out_dims = NumpyBackend._merge_dims(a, b)
        res = table[kind](NumpyBackend._to_dims(a, out_dims), NumpyBackend._to_dims(b, out_dims))
        res = numpy.asarray(res)
        src = a if a._dims == out_dims or not b._dims else b
        return Tensor("numpy_%s" % kind, dims=list(out_dims), dtype=NumpyBackend.get_dtype_name_raw(res), raw_tensor=res,
                      sparse_dim=src.sparse_dim if table is _BIN and res.dtype.kind in "iu" else None)

    @staticmethod
    def compare(a, kind: str, b) -> Tensor:
        """named-dim comparison"""
        return NumpyBackend._binary(a, kind, b, _CMP)

    @staticmethod
    def combine(a, kind: str, b) -> Tensor:
        """named-dim binary op"""
        return NumpyBackend._binary(a, kind, b, _BIN)

    @staticmethod
    def where(cond: Tensor, true_, false_) -> Tensor:
        """select"""
        ts = [t for t in (cond, true_, false_) if isinstance(t, Tensor)]
        out_dims: Tuple[Dim, ...] = ()
        for t in ts:
            out_dims = NumpyBackend._merge_dims(Tensor("tmp", dims=list(out_dims), dtype="bool"), t) if out_dims else tuple(t._dims)
        raws = [NumpyBackend._to_dims(t, out_dims) if isinstance(t, Tensor) else t for t in (cond, true_, false_)]
        res = numpy.where(*raws)
        return Tensor("where", dims=list(out_dims), dtype=NumpyBackend.get_dtype_name_raw(res), raw_tensor=res)

    @staticmethod
    def range_over_dim(dim: Dim, *, dtype: Optional[str] = None, device: Optional[str] = None) -> Tensor:
        """0 .. dim-1 along dim"""
        n = dim.dimension if dim.dimension is not None else int(numpy.max(numpy.asarray(dim.dyn_size_ext.raw_tensor)))
        arr = numpy.arange(n, dtype=dtype or "int32")
        return Tensor("range", dims=[dim], dtype=arr.dtype.name, sparse_dim=dim, raw_tensor=arr)

    @staticmethod
    def reduce(source: Tensor, *, mode: str, axis: Union[Dim, Sequence[Dim]], use_mask: bool = True) -> Tensor:
        """sum / max / min / mean / any / all / argmax / argmin / logsumexp over axis, padded frames ignored"""
        axes = [axis] if isinstance(axis, Dim) else list(axis)
        raw = numpy.asarray(source._raw_tensor)
        idxs = tuple(source._dims.index(d) for d in axes)
        count = None
        if use_mask:
            for d in axes:
                if d.dyn_size_ext is not None and d.dyn_size_ext.dims:
                    sizes = d.dyn_size_ext
                    rng = NumpyBackend.range_over_dim(d)
                    mask = NumpyBackend.compare(rng, "<", Tensor("sizes", dims=list(sizes.dims), dtype="int32", raw_tensor=numpy.asarray(sizes.raw_tensor)))
                    m = NumpyBackend._to_dims(mask, source._dims)
                    neutral = {"sum": 0, "mean": 0, "max": -numpy.inf, "argmax": -numpy.inf, "logsumexp": -numpy.inf, "min": numpy.inf,
                               "argmin": numpy.inf, "any": False, "all": True}[mode]
                    if raw.dtype.kind in "iu" and not numpy.isfinite(neutral):
                        neutral = numpy.iinfo(raw.dtype).min if neutral < 0 else numpy.iinfo(raw.dtype).max
                    raw = numpy.where(m, raw, numpy.asarray(neutral, dtype=raw.dtype))
                    if mode == "mean":
                        count = numpy.sum(numpy.broadcast_to(m, raw.shape), axis=idxs)
        dims = [d for i, d in enumerate(source._dims) if i not in idxs]
        if mode in ("argmax", "argmin"):
            assert len(idxs) == 1
            res = (numpy.argmax if mode == "argmax" else numpy.argmin)(raw, axis=idxs[0]).astype("int32")
            return Tensor("reduce", dims=dims, dtype="int32", sparse_dim=axes[0], raw_tensor=res)
        if mode == "mean":
            res = numpy.sum(raw, axis=idxs) / count if count is not None else numpy.mean(raw, axis=idxs)
        elif mode == "logsumexp":
            mx = numpy.max(raw, axis=idxs, keepdims=True)
            mx = numpy.where(numpy.isfinite(mx), mx, 0)
            res = numpy.log(numpy.sum(numpy.exp(raw - mx), axis=idxs)) + numpy.squeeze(mx, axis=idxs)
        else:
            res = {"sum": numpy.sum, "max": numpy.max, "min": numpy.min, "any": numpy.any, "all": numpy.all}[mode](raw, axis=idxs)
        res = numpy.asarray(res)
        return Tensor("reduce", dims=dims, dtype=NumpyBackend.get_dtype_name_raw(res), raw_tensor=res)
