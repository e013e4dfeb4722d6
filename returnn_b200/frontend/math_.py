"""
Element-wise math: comparisons, binary arithmetic with broadcasting by dim identity, unary functions, activations,
softmax family.

Parity: returnn/frontend/math_.py:1-709 (compare/combine, activations, gating :665),
softmax semantics returnn/torch/frontend/_backend.py:631-690 (masking of padded frames with a large negative value).
"""

from __future__ import annotations
from typing import Optional, Sequence, Union, Callable
import math as _math
import numpy
import torch
from . import _numpy_backend as _np
import torch.nn.functional as F
from ..tensor import Tensor, Dim
from ..tensor.utils import host_to_device
from ._utils import wrap, merge_dims_for_broadcast, convert_to_tensor, torch_dtype, dtype_name
from ..utils.basic import NotSpecified

__all__ = [
    "compare", "compare_bc", "combine", "combine_bc", "equal", "less", "less_equal", "greater", "greater_equal",
    "not_equal", "add", "sub", "mul", "true_divide", "floor_divide", "ceil_divide", "neg", "reciprocal", "mod", "pow",
    "squared_difference", "logical_and", "logical_or", "logical_not", "opt_logical_or", "opt_logical_and",
    "is_finite", "is_infinite", "is_neg_infinite", "maximum", "minimum", "clip_by_value", "lerp", "identity", "exp",
    "expm1", "log", "safe_log", "log1p", "sqrt", "rsqrt", "square", "abs", "tanh", "sigmoid", "log_sigmoid", "sin",
    "cos", "ceil", "floor", "round", "relu", "relu_square", "elu", "selu", "silu", "swish", "gelu", "softplus", "softmax",
    "log_softmax", "gating", "glu", "sign", "erf", "leaky_relu", "hardtanh", "log_add_exp",
]

_CMP = {
    "==": torch.eq, "eq": torch.eq, "equal": torch.eq,
    "!=": torch.ne, "<>": torch.ne, "not_equal": torch.ne, "ne": torch.ne,
    "<": torch.lt, "less": torch.lt, "lt": torch.lt,
    "<=": torch.le, "less_equal": torch.le, "le": torch.le,
    ">": torch.gt, "greater": torch.gt, "gt": torch.gt,
    ">=": torch.ge, "greater_equal": torch.ge, "ge": torch.ge,
}


def _floordiv(a, b):
    return torch.div(a, b, rounding_mode="floor")


def _pow(a, b):
    return torch.pow(a, b)


def _sqdiff(a, b):
    d = a - b
    return d * d


_BIN = {
    "+": torch.add, "add": torch.add,
    "-": torch.sub, "sub": torch.sub,
    "*": torch.mul, "mul": torch.mul,
    "/": torch.true_divide, "truediv": torch.true_divide, "true_divide": torch.true_divide,
    "//": _floordiv, "floordiv": _floordiv, "floor_divide": _floordiv,
    "%": torch.remainder, "mod": torch.remainder,
    "**": _pow, "pow": _pow,
    "max": torch.maximum, "maximum": torch.maximum,
    "min": torch.minimum, "minimum": torch.minimum,
    "logical_and": torch.logical_and, "logical_or": torch.logical_or,
    "squared_difference": _sqdiff,
    "logaddexp": torch.logaddexp,
}


def _prep_bin(a, b, allow_broadcast_all_sources, dim_order):
    a_is_t = isinstance(a, Tensor)
    b_is_t = isinstance(b, Tensor)
    if not a_is_t and not b_is_t:
        a = convert_to_tensor(a)
        a_is_t = True
    if not b_is_t:
        b = convert_to_tensor(b, like=a)
    elif not a_is_t:
        a = convert_to_tensor(a, like=b)
    ad, bd = a._dims, b._dims
    if ad == bd:
        out_dims = ad
        ra, rb = a._raw_tensor, b._raw_tensor
    else:
        out_dims = merge_dims_for_broadcast(a, b)
        if allow_broadcast_all_sources is False and out_dims != ad and out_dims != bd:
            if set(out_dims) != set(ad) and set(out_dims) != set(bd):
                raise ValueError("combine/compare: %r and %r: not allow_broadcast_all_sources" % (a, b))
        ra = a.copy_compatible_to_dims_raw(out_dims) if ad else a._raw_tensor
        rb = b.copy_compatible_to_dims_raw(out_dims) if bd else b._raw_tensor
    if dim_order is not None and tuple(dim_order) != tuple(out_dims) and set(dim_order) == set(out_dims):
        ra = a.copy_compatible_to_dims_raw(dim_order) if ad else ra
        rb = b.copy_compatible_to_dims_raw(dim_order) if bd else rb
        out_dims = tuple(dim_order)
    return a, b, ra, rb, out_dims


def compare(a, kind: str, b, *, allow_broadcast_all_sources: Optional[bool] = None, dim_order: Optional[Sequence[Dim]] = None) -> Tensor:
    """
    :param kind: "==", "!=", "<", "<=", ">", ">=" or the word forms
    :return: bool tensor, dims = union of the operand dims
    """
    if _np.is_numpy(a) or _np.is_numpy(b):
        return _np.NumpyBackend.compare(a, kind, b)
    a, b, ra, rb, out_dims = _prep_bin(a, b, allow_broadcast_all_sources, dim_order)
    fn = _CMP.get(kind)
    if fn is None:
        raise ValueError("compare: invalid kind %r" % kind)
    if ra.device != rb.device:
        # a host operand (scalar, sizes, a step counter of a decoder state) follows the device operand
        if not rb.ndim or (rb.device.type == "cpu" and ra.device.type != "cpu"):
            rb = host_to_device(rb, ra.device)
        elif not ra.ndim or ra.device.type == "cpu":
            ra = host_to_device(ra, rb.device)
    return wrap(fn(ra, rb), out_dims, name="compare")


def combine(a, kind: str, b, *, allow_broadcast_all_sources: Optional[bool] = None, dim_order: Optional[Sequence[Dim]] = None) -> Tensor:
    """
    :param kind: "+", "-", "*", "/", "//", "%", "**", "max", "min", "logical_and", "logical_or", "squared_difference"
    :return: dims = union of the operand dims
    """
    if _np.is_numpy(a) or _np.is_numpy(b):
        return _np.NumpyBackend.combine(a, kind, b)
    a, b, ra, rb, out_dims = _prep_bin(a, b, allow_broadcast_all_sources, dim_order)
    fn = _BIN.get(kind)
    if fn is None:
        raise ValueError("combine: invalid kind %r" % kind)
    if ra.device != rb.device:
        # a host operand (scalar, sizes, a step counter of a decoder state) follows the device operand
        if not rb.ndim or (rb.device.type == "cpu" and ra.device.type != "cpu"):
            rb = host_to_device(rb, ra.device)
        elif not ra.ndim or ra.device.type == "cpu":
            ra = host_to_device(ra, rb.device)
    res = fn(ra, rb)
    src = a if a._dims == out_dims or not b._dims else b
    return wrap(res, out_dims, name="combine", like=src)


compare_bc = compare
combine_bc = combine


def log_add_exp(a: Tensor, b: Tensor) -> Tensor:
    """``log(exp(a) + exp(b))`` computed stably (sums of log probabilities, e.g. in beam search); see also ``reduce_logsumexp``"""
    return combine(a, "logaddexp", b)


def equal(a, b):
    """a == b"""
    return compare(a, "==", b)


def not_equal(a, b):
    """a != b"""
    return compare(a, "!=", b)


def less(a, b):
    """a < b"""
    return compare(a, "<", b)


def less_equal(a, b):
    """a <= b"""
    return compare(a, "<=", b)


def greater(a, b):
    """a > b"""
    return compare(a, ">", b)


def greater_equal(a, b):
    """a >= b"""
    return compare(a, ">=", b)


def add(a, b):
    """a + b"""
    return combine(a, "+", b)


def sub(a, b):
    """a - b"""
    return combine(a, "-", b)


def mul(a, b):
    """a * b"""
    return combine(a, "*", b)


def true_divide(a, b):
    """a / b"""
    return combine(a, "/", b)


def floor_divide(a, b):
    """a // b"""
    return combine(a, "//", b)


def ceil_divide(a, b):
    """ceil(a / b) for ints"""
    return neg(floor_divide(neg(a), b))


def mod(a, b):
    """a % b"""
    return combine(a, "%", b)


def pow(a, b):
    """a ** b"""
    return combine(a, "**", b)


def squared_difference(a, b):
    """(a - b) ** 2"""
    return combine(a, "squared_difference", b)


def logical_and(a, b):
    """a and b"""
    return combine(a, "logical_and", b)


def logical_or(a, b):
    """a or b"""
    return combine(a, "logical_or", b)


def opt_logical_or(a, b):
    """logical_or where python bools short-circuit"""
    if isinstance(a, bool):
        return True if a else b
    if isinstance(b, bool):
        return True if b else a
    return logical_or(a, b)


def opt_logical_and(a, b):
    """logical_and where python bools short-circuit"""
    if isinstance(a, bool):
        return b if a else False
    if isinstance(b, bool):
        return a if b else False
    return logical_and(a, b)


def maximum(a, b, *other):
    """element-wise max"""
    res = combine(a, "max", b)
    for o in other:
        res = combine(res, "max", o)
    return res


def minimum(a, b, *other):
    """element-wise min"""
    res = combine(a, "min", b)
    for o in other:
        res = combine(res, "min", o)
    return res


def clip_by_value(x: Tensor, clip_value_min, clip_value_max, *, allow_broadcast_all_sources: bool = False) -> Tensor:
    """clamp"""
    if not isinstance(clip_value_min, Tensor) and not isinstance(clip_value_max, Tensor):
        return wrap(torch.clamp(x._raw_tensor, clip_value_min, clip_value_max), x._dims, like=x)
    return minimum(maximum(x, clip_value_min), clip_value_max)


def lerp(start: Tensor, end: Tensor, weight) -> Tensor:
    """start + weight * (end - start)"""
    return start + weight * (end - start)


def _unary(fn: Callable, name: str):
    def f(a: Tensor) -> Tensor:
        return wrap(fn(a._raw_tensor), a._dims, name=name, like=a)

    f.__name__ = name
    f.__qualname__ = name
    f.__doc__ = "element-wise %s" % name
    return f


def identity(x: Tensor) -> Tensor:
    """x"""
    return x


neg = _unary(torch.neg, "neg")
logical_not = _unary(torch.logical_not, "logical_not")
reciprocal = _unary(torch.reciprocal, "reciprocal")
exp = _unary(torch.exp, "exp")
expm1 = _unary(torch.expm1, "expm1")
log = _unary(torch.log, "log")
log1p = _unary(torch.log1p, "log1p")
sqrt = _unary(torch.sqrt, "sqrt")
rsqrt = _unary(torch.rsqrt, "rsqrt")
square = _unary(torch.square, "square")
abs = _unary(torch.abs, "abs")
tanh = _unary(torch.tanh, "tanh")
sigmoid = _unary(torch.sigmoid, "sigmoid")
log_sigmoid = _unary(F.logsigmoid, "log_sigmoid")
sin = _unary(torch.sin, "sin")
cos = _unary(torch.cos, "cos")
ceil = _unary(torch.ceil, "ceil")
floor = _unary(torch.floor, "floor")
round = _unary(torch.round, "round")
relu = _unary(torch.relu, "relu")
elu = _unary(F.elu, "elu")
selu = _unary(F.selu, "selu")
silu = _unary(F.silu, "silu")
swish = silu
gelu = _unary(F.gelu, "gelu")
softplus = _unary(F.softplus, "softplus")
sign = _unary(torch.sign, "sign")
erf = _unary(torch.erf, "erf")
is_finite = _unary(torch.isfinite, "is_finite")
is_infinite = _unary(torch.isinf, "is_infinite")
is_neg_infinite = _unary(torch.isneginf, "is_neg_infinite")


def relu_square(x: Tensor) -> Tensor:
    """relu(x) ** 2"""
    return wrap(torch.square(torch.relu(x._raw_tensor)), x._dims, like=x)


def leaky_relu(x: Tensor, negative_slope: float = 0.01) -> Tensor:
    """leaky relu"""
    return wrap(F.leaky_relu(x._raw_tensor, negative_slope), x._dims, like=x)


def hardtanh(x: Tensor, min_val: float = -1.0, max_val: float = 1.0) -> Tensor:
    """clamp to [min_val, max_val]"""
    return wrap(F.hardtanh(x._raw_tensor, min_val, max_val), x._dims, like=x)


def safe_log(x: Tensor, *, eps: Optional[float] = None) -> Tensor:
    """log(max(x, eps)); default eps is the smallest normal of the dtype"""
    if eps is None:
        eps = {"float16": 6e-08, "bfloat16": 9.1835e-41, "float32": 1.4013e-45, "float64": 4.94066e-324}[x.dtype]
    return wrap(torch.log(torch.clamp_min(x._raw_tensor, eps)), x._dims, like=x)


def _softmax_impl(x: Tensor, axis: Dim, use_mask: bool, log_: bool) -> Tensor:
    from ._utils import axis_of

    ax = axis_of(x, axis)
    raw = x._raw_tensor
    if use_mask and axis.is_dynamic() and axis.need_masking() and axis.is_dynamic_seq_length():
        mask = axis.get_mask(device=raw.device).copy_compatible_to_dims_raw(x._dims)
        neg = -1e30 if raw.dtype in (torch.float32, torch.float64) else -3e4 if raw.dtype == torch.float16 else -1e30
        raw = torch.where(mask, raw, torch.full((), neg, dtype=raw.dtype, device=raw.device))
    out = F.log_softmax(raw, dim=ax) if log_ else F.softmax(raw, dim=ax)
    return wrap(out, x._dims, like=x)


def softmax(x: Tensor, *, axis: Dim, use_mask: bool = True) -> Tensor:
    """softmax over axis; padded frames of a dynamic axis get probability 0"""
    return _softmax_impl(x, axis, use_mask, False)


def log_softmax(x: Tensor, *, axis: Dim, use_mask: bool = True) -> Tensor:
    """log softmax over axis"""
    return _softmax_impl(x, axis, use_mask, True)


def gating(x: Tensor, *, axis: Optional[Dim] = None, gate_func=sigmoid, act_func=identity, out_dim: Optional[Dim] = None):
    """
    Split ``axis`` in two halves a, b; return ``act_func(a) * gate_func(b)`` and the new dim.
    With the defaults this is GLU.
    """
    from .array_ import split

    if axis is None:
        axis = x.feature_dim
    assert axis is not None and axis.dimension % 2 == 0
    if out_dim is None:
        out_dim = axis.div_left(2)
    a, b = split(x, axis=axis, out_dims=[out_dim, out_dim])
    return act_func(a) * gate_func(b), out_dim


def glu(x: Tensor, *, axis: Optional[Dim] = None, out_dim: Optional[Dim] = None):
    """gated linear unit"""
    return gating(x, axis=axis, out_dim=out_dim)
