"""
``Dim``: a named axis. Static (``dimension`` is an int) or dynamic (``dimension is None``; the per-sequence sizes
are in ``dyn_size_ext``, a :class:`Tensor` of shape ``[]`` or ``[batch]`` kept on the host).

Identity semantics: two ``Dim`` objects are the same axis only if they are the same object (or were declared the same
with :func:`Dim.declare_same_as`). Dim arithmetic (``a + b``, ``2 * a``, ``a.ceildiv_right(6)``) is memoised, so the
same expression gives the same ``Dim`` object and tensors built from it stay compatible.

Parity: returnn/tensor/dim.py:38, returnn/tensor/_dim_extra.py (dim math, masks, dyn sizes, ``capacity`` /
``bounded_by`` for static-shape regimes), returnn/tensor/marked_dim.py.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union, TYPE_CHECKING
import numpy

if TYPE_CHECKING:
    from .tensor import Tensor

__all__ = ["Dim", "batch_dim", "single_step_dim", "VerifyOutShapeException", "DimTypes"]


class DimTypes:
    """kind of a dim"""

    class _Kind:
        def __init__(self, name):
            self.name = name

        def __repr__(self):
            return "<%s>" % self.name

        def __reduce__(self):
            return getattr, (DimTypes, {"unspecified": "Unspecified", "batch": "Batch", "spatial": "Spatial",
                                        "feature": "Feature"}[self.name])

    Unspecified = None
    Batch = _Kind("batch")
    Spatial = _Kind("spatial")
    Time = Spatial
    Feature = _Kind("feature")
    Types = (Batch, Spatial, Feature)


class VerifyOutShapeException(Exception):
    """raised by Tensor.verify_out_shape"""


class _DimOp:
    """how a derived dim was computed"""

    __slots__ = ("kind", "inputs", "attribs")

    def __init__(self, kind: str, inputs: Sequence[Union["Dim", int]], attribs: Optional[Dict[str, Any]] = None):
        self.kind = kind
        self.inputs = tuple(inputs)
        self.attribs = attribs

    def key(self):
        """memo key"""
        return (
            self.kind,
            tuple(id(x.get_same_base()) if isinstance(x, Dim) else ("c", x) for x in self.inputs),
            tuple(sorted(self.attribs.items())) if self.attribs else None,
        )

    def __repr__(self):
        return "DimOp(%s, %r)" % (self.kind, self.inputs)


_derived_cache: Dict[Any, "Dim"] = {}


def _apply_int_op(kind: str, a, b):
    """a, b: python ints or numpy arrays / torch tensors"""
    if kind == "add":
        return a + b
    if kind == "sub":
        return a - b
    if kind == "mul":
        return a * b
    if kind == "floordiv":
        return a // b
    if kind == "ceildiv":
        return -(-a // b)
    if kind == "max":
        return numpy.maximum(a, b) if isinstance(a, numpy.ndarray) or isinstance(b, numpy.ndarray) else max(a, b)
    raise ValueError(kind)


class Dim:
    """
    One axis of a :class:`Tensor`.
    """

    Types = DimTypes

    def __init__(
        self,
        dimension: Union[int, None, "Tensor"],
        *,
        name: Optional[str] = None,
        kind=DimTypes.Unspecified,
        dyn_size_ext: Optional["Tensor"] = None,
        description: Optional[str] = None,
        capacity: Optional[int] = None,
        bounded_by: Optional[int] = None,
        vocab=None,
        derived_from_op: Optional[_DimOp] = None,
        auto_generated: bool = False,
        **_ignored,
    ):
        """
        :param dimension: int for static; None for dynamic; a Tensor (scalar or [batch]) gives the dynamic sizes
        :param name: for humans; not part of identity
        :param kind: batch / spatial / feature
        :param dyn_size_ext: sizes of a dynamic dim
        :param capacity: upper bound on the dim value used to allocate static buffers (CUDA-graph regime)
        :param bounded_by: like capacity but a hard promise about the data
        :param vocab: optional vocabulary for sparse dims
        """
        if dimension is not None and not isinstance(dimension, (int, numpy.integer)):
            from .tensor import Tensor

            assert isinstance(dimension, Tensor), "Dim: invalid dimension %r" % (dimension,)
            assert dyn_size_ext is None
            dyn_size_ext = dimension
            dimension = None
        elif dimension is not None:
            assert isinstance(dimension, (int, numpy.integer)), "Dim: invalid dimension %r" % (dimension,)
            dimension = int(dimension)
        self.dimension: Optional[int] = dimension
        self.size = dimension
        self.name = name or description
        self.kind = kind
        self.capacity = capacity
        self.bounded_by = bounded_by
        self.vocab = vocab
        self.derived_from_op = derived_from_op
        self.auto_generated = auto_generated
        self._dyn_size_ext: Optional["Tensor"] = None
        self._same_as: Optional["Dim"] = None
        self._mask_cache: Dict[Any, "Tensor"] = {}
        self._dim_value_cache: Optional[int] = None
        self._size_tensor_cache: Dict[Any, "Tensor"] = {}
        self._version = 0  # bumped whenever the sizes change
        self._derived_versions = None  # versions of the op inputs the sizes were computed from
        self.match_priority = 0
        if dyn_size_ext is not None:
            self.dyn_size_ext = dyn_size_ext

    # -- identity ---------------------------------------------------------------------------------
    def get_same_base(self) -> "Dim":
        """root of the declare_same_as chain"""
        d = self
        while d._same_as is not None:
            d = d._same_as
        return d

    def declare_same_as(self, other: "Dim"):
        """from now on, self and other are the same axis"""
        a, b = self.get_same_base(), other.get_same_base()
        if a is b:
            return
        if a.dimension is not None and b.dimension is not None:
            assert a.dimension == b.dimension, "declare_same_as: %r vs %r" % (self, other)
        a._same_as = b
        if b._dyn_size_ext is None and a._dyn_size_ext is not None:
            b._dyn_size_ext = a._dyn_size_ext
        if b.dimension is None and a.dimension is not None:
            b.dimension = b.size = a.dimension

    def __eq__(self, other):
        if not isinstance(other, Dim):
            return False
        return self.get_same_base() is other.get_same_base()

    def __ne__(self, other):
        return not (self == other)

    def __hash__(self):
        return id(self.get_same_base())

    def is_equal(self, other: "Dim", **_kwargs) -> bool:
        """same axis"""
        return self == other

    def __repr__(self):
        return "Dim{%s}" % self.short_repr()

    def short_repr(self) -> str:
        """'name'(size)"""
        if self.is_batch_dim():
            return "B"
        d = self.get_same_base()
        size = "?" if d.dimension is None else str(d.dimension)
        return "%r(%s)" % (self.name or "unnamed", size)

    def __copy__(self):
        return self

    def __deepcopy__(self, memo=None):
        return self

    def __reduce__(self):
        if self is batch_dim:
            return _get_global_dim, ("batch_dim",)
        if self is single_step_dim:
            return _get_global_dim, ("single_step_dim",)
        return _make_dim, (self.dimension, self.name, self.kind, self.capacity, self.bounded_by, self.vocab)

    def copy(self, same_as_self: bool = True, description: Optional[str] = None, **kwargs) -> "Dim":
        """
        :param same_as_self: if False, a new distinct axis with the same size info
        """
        if same_as_self:
            return self
        d = Dim(
            self.dimension,
            name=description or self.name,
            kind=self.kind,
            capacity=self.capacity,
            bounded_by=self.bounded_by,
            vocab=self.vocab,
        )
        if self.dyn_size_ext is not None:
            d.dyn_size_ext = self.dyn_size_ext
        return d

    # -- kinds -------------------------------------------------------------------------------------
    def is_batch_dim(self) -> bool:
        """batch axis"""
        return self.get_same_base().kind is DimTypes.Batch

    def is_feature_dim(self) -> bool:
        """feature axis"""
        return self.kind is DimTypes.Feature

    def is_spatial_dim(self) -> bool:
        """spatial axis"""
        return self.kind is DimTypes.Spatial

    def is_static(self) -> bool:
        """fixed size"""
        return self.get_same_base().dimension is not None

    def is_dynamic(self) -> bool:
        """size known only with data"""
        return self.get_same_base().dimension is None

    def is_dynamic_seq_length(self) -> bool:
        """dynamic with per-sequence sizes (not a scalar)"""
        d = self.dyn_size_ext
        return d is not None and len(d.dims) > 0

    def need_masking(self) -> bool:
        """whether padded frames exist in principle"""
        if self.is_static():
            return False
        if self.capacity is not None:
            return True
        d = self.dyn_size_ext
        if d is None:
            return True
        return len(d.dims) > 0

    def is_dim_known(self) -> bool:
        """static or sizes are set"""
        if self.is_batch_dim():
            return True
        return self.is_static() or self.dyn_size_ext is not None

    # -- dynamic sizes -----------------------------------------------------------------------------
    @property
    def dyn_size_ext(self) -> Optional["Tensor"]:
        """sizes as Tensor, shape [] or [batch...]; computed lazily for derived dims"""
        base = self.get_same_base()
        if base.derived_from_op is not None and base.dimension is None:
            base._maybe_refresh_derived()
        return base._dyn_size_ext

    @dyn_size_ext.setter
    def dyn_size_ext(self, value: Optional["Tensor"]):
        base = self.get_same_base()
        base._dyn_size_ext = value
        base._invalidate()
        if base.derived_from_op is not None:
            base._derived_versions = base._input_versions()

    def _invalidate(self):
        self._mask_cache.clear()
        self._size_tensor_cache.clear()
        self._dim_value_cache = None
        self._version += 1

    def _current_version(self) -> int:
        base = self.get_same_base()
        if base.derived_from_op is not None and base.dimension is None:
            base._maybe_refresh_derived()
        return base._version

    def _input_versions(self):
        return tuple(x._current_version() for x in self.derived_from_op.inputs if isinstance(x, Dim))

    def _maybe_refresh_derived(self):
        """sizes of a derived dim follow the sizes of the dims it was computed from"""
        vers = self._input_versions()
        if vers == self._derived_versions and self._dyn_size_ext is not None:
            return
        self._dyn_size_ext = None
        self._compute_dyn_size_from_op()
        self._derived_versions = vers
        self._invalidate()

    @property
    def dyn_size(self):
        """raw sizes"""
        d = self.dyn_size_ext
        return None if d is None else d.raw_tensor

    @dyn_size.setter
    def dyn_size(self, value):
        from .tensor import Tensor

        if value is None:
            self.dyn_size_ext = None
            return
        ndim = getattr(value, "ndim", 0)
        dims = [batch_dim] if ndim == 1 else []
        self.dyn_size_ext = Tensor("%s:size" % (self.name or "dim"), dims=dims, dtype="int32", raw_tensor=value)

    def reset_eager(self):
        """forget data-dependent state"""
        self.reset_raw()

    def reset_raw(self, only_self: bool = False):
        """drop raw size tensors and caches"""
        base = self.get_same_base()
        base._dyn_size_ext = None
        base._derived_versions = None
        base._invalidate()

    def _compute_dyn_size_from_op(self):
        from .tensor import Tensor

        op = self.derived_from_op
        vals = []
        dims: List[Dim] = []
        for x in op.inputs:
            if isinstance(x, Dim):
                if x.is_static():
                    vals.append(x.dimension)
                else:
                    ext = x.dyn_size_ext
                    if ext is None or ext.raw_tensor is None:
                        return
                    vals.append(ext)
                    for d in ext.dims:
                        if d not in dims:
                            dims.append(d)
            else:
                vals.append(x)
        raws = []
        for v in vals:
            if isinstance(v, Tensor):
                r = v.copy_compatible_to_dims_raw(dims)
                raws.append(r)
            else:
                raws.append(v)
        if op.kind in ("add", "sub", "mul", "floordiv", "ceildiv"):
            res = raws[0]
            for r in raws[1:]:
                res = _apply_int_op(op.kind, res, r)
        elif op.kind == "pad":
            res = raws[0] + op.attribs["left"] + op.attribs["right"]
        elif op.kind == "conv":
            # out = ceildiv(in - (fs-1)*dil, stride) for valid; ceildiv(in, stride) for same
            a = op.attribs
            res = raws[0]
            if a["padding"] == "valid":
                res = res - (a["filter_size"] - 1) * a["dilation"]
            elif isinstance(a["padding"], int):
                res = res + 2 * a["padding"] - (a["filter_size"] - 1) * a["dilation"]
            res = -(-res // a["stride"])
            import torch

            if isinstance(res, torch.Tensor):
                res = res.clamp(min=0)
            else:
                res = numpy.maximum(res, 0)
        else:
            return
        self._dyn_size_ext = Tensor("%s:size" % (self.name or "dim"), dims=dims, dtype="int32", raw_tensor=res)

    def get_dim_value(self) -> int:
        """static size, or max over the dynamic sizes"""
        base = self.get_same_base()
        if base.dimension is not None:
            return base.dimension
        if base.derived_from_op is not None:
            base._maybe_refresh_derived()
        if base._dim_value_cache is not None:
            return base._dim_value_cache
        if base.capacity is not None and self.dyn_size_ext is not None and getattr(self.dyn_size_ext.raw_tensor, "is_cuda", False):
            # static-shape regime (captured CUDA graphs): the tensors have the capacity as their extent and the lengths live on
            # the device, where reading their maximum would synchronise
            return base.capacity
        ext = self.dyn_size_ext
        if ext is None or ext.raw_tensor is None:
            raise Exception("%r: dynamic size unknown" % self)
        raw = ext.raw_tensor
        v = int(raw.max()) if getattr(raw, "ndim", 0) > 0 and raw.numel() > 0 else (int(raw) if getattr(raw, "ndim", 0) == 0 else 0)
        base._dim_value_cache = v
        return v

    def get_dim_value_tensor(self):
        """dim value as scalar Tensor or int"""
        if self.is_static():
            return self.dimension
        from .tensor import Tensor
        import torch

        return Tensor("%s:max" % self.name, dims=[], dtype="int32", raw_tensor=torch.tensor(self.get_dim_value(), dtype=torch.int32))

    def get_size_tensor(self, device=None) -> "Tensor":
        """sizes as Tensor (scalar for static dims)"""
        from .tensor import Tensor
        import torch

        if self.is_static():
            return Tensor("%s:size" % self.name, dims=[], dtype="int32", raw_tensor=torch.tensor(self.dimension, dtype=torch.int32))
        ext = self.dyn_size_ext
        assert ext is not None, "%r: no sizes" % self
        if device is None:
            return ext
        key = str(device)
        base = self.get_same_base()
        if key not in base._size_tensor_cache:
            from .utils import host_to_device

            base._size_tensor_cache[key] = ext.copy_with_raw(host_to_device(ext.raw_tensor, device))
        return base._size_tensor_cache[key]

    def get_dyn_size_ext_for_device(self, device=None) -> "Tensor":
        """alias of get_size_tensor for dynamic dims"""
        return self.get_size_tensor(device=device)

    def get_mask(self, *, dim_order: Optional[Sequence["Dim"]] = None, device=None) -> "Tensor":
        """
        :return: bool Tensor, True inside the sequence. Dims are ``dyn_size_ext.dims + [self]`` (or dim_order).
        """
        from .tensor import Tensor
        import torch

        assert self.is_dynamic(), "%r: mask only for dynamic dims" % self
        ext = self.dyn_size_ext
        assert ext is not None and ext.raw_tensor is not None, "%r: sizes unknown" % self
        base = self.get_same_base()
        key = (str(device), tuple(id(d.get_same_base()) for d in dim_order) if dim_order else None)
        if key in base._mask_cache:
            return base._mask_cache[key]
        sizes = ext.raw_tensor
        if not isinstance(sizes, torch.Tensor):
            sizes = torch.as_tensor(numpy.asarray(sizes))
        max_len = self.get_dim_value()
        if device is not None:
            from .utils import host_to_device

            sizes = host_to_device(sizes, device)
        rng = torch.arange(max_len, device=sizes.device, dtype=sizes.dtype)
        mask_raw = rng.reshape([1] * sizes.ndim + [max_len]) < sizes.unsqueeze(-1)
        mask = Tensor("%s:mask" % (self.name or "dim"), dims=list(ext.dims) + [self], dtype="bool", raw_tensor=mask_raw)
        if dim_order:
            mask = mask.copy_transpose_to_dims([d for d in dim_order if d in mask.dims])
        base._mask_cache[key] = mask
        return mask

    def get_for_batch_ctx(self, *args, **kwargs) -> "Dim":
        """there is a single eager context here"""
        return self

    def get_dim_value_ceiled(self) -> int:
        """capacity if set (static-shape regime) else the dim value"""
        if self.capacity is not None:
            return self.capacity
        return self.get_dim_value()

    # -- arithmetic --------------------------------------------------------------------------------
    @staticmethod
    def _derive(kind: str, inputs: Sequence[Union["Dim", int]], attribs=None, name: Optional[str] = None) -> "Dim":
        simp = Dim._simplify(kind, inputs)
        if simp is not None:
            return simp
        op = _DimOp(kind, inputs, attribs)
        key = op.key()
        res = _derived_cache.get(key)
        if res is not None:
            return res
        dims_in = [x for x in inputs if isinstance(x, Dim)]
        all_static = all(d.is_static() for d in dims_in)
        dimension = None
        if all_static:
            vals = [x.dimension if isinstance(x, Dim) else x for x in inputs]
            if kind in ("add", "sub", "mul", "floordiv", "ceildiv"):
                dimension = vals[0]
                for v in vals[1:]:
                    dimension = _apply_int_op(kind, dimension, v)
            elif kind == "pad":
                dimension = vals[0] + attribs["left"] + attribs["right"]
            elif kind == "conv":
                dimension = vals[0]
                if attribs["padding"] == "valid":
                    dimension -= (attribs["filter_size"] - 1) * attribs["dilation"]
                elif isinstance(attribs["padding"], int):
                    dimension += 2 * attribs["padding"] - (attribs["filter_size"] - 1) * attribs["dilation"]
                dimension = max(-(-dimension // attribs["stride"]), 0)
        kind_ = dims_in[0].kind if dims_in else DimTypes.Unspecified
        if kind_ is DimTypes.Batch:
            kind_ = DimTypes.Spatial
        if name is None:
            sym = {"add": "+", "sub": "-", "mul": "*", "floordiv": "//", "ceildiv": "⌈/⌉"}.get(kind, kind)
            name = sym.join((x.name or "?") if isinstance(x, Dim) else str(x) for x in inputs)
            if kind in ("pad", "conv"):
                name = "%s(%s)" % (kind, name)
        res = Dim(dimension, name=name, kind=kind_, derived_from_op=op, auto_generated=True)
        caps = [d.capacity for d in dims_in]
        if dimension is None and all(c is not None for c in caps) and kind in ("add", "sub", "mul", "floordiv", "ceildiv"):
            cap = caps[0] if isinstance(inputs[0], Dim) else inputs[0]
            it = iter(caps)
            vals = [next(it) if isinstance(x, Dim) else x for x in inputs]
            cap = vals[0]
            for v in vals[1:]:
                cap = _apply_int_op(kind, cap, v)
            res.capacity = int(cap)
        elif dimension is None and caps and caps[0] is not None and kind == "pad":
            res.capacity = int(caps[0]) + attribs["left"] + attribs["right"]
        elif dimension is None and caps and caps[0] is not None and kind == "conv":
            cap = int(caps[0])
            if attribs["padding"] == "valid":
                cap -= (attribs["filter_size"] - 1) * attribs["dilation"]
            elif isinstance(attribs["padding"], int):
                cap += 2 * attribs["padding"] - (attribs["filter_size"] - 1) * attribs["dilation"]
            res.capacity = max(-(-cap // attribs["stride"]), 0)
        _derived_cache[key] = res
        return res

    @staticmethod
    def _simplify(kind: str, inputs) -> Optional["Dim"]:
        """inverse operations cancel: (c*d)//c -> d, (a+b)-b -> a, (a-b)+b -> a"""
        if len(inputs) != 2 or not isinstance(inputs[0], Dim):
            return None
        a, b = inputs
        op = a.get_same_base().derived_from_op
        if op is None or len(op.inputs) != 2:
            return None
        x, y = op.inputs

        def same(p, q):
            if isinstance(p, Dim) and isinstance(q, Dim):
                return p == q
            if isinstance(p, Dim) or isinstance(q, Dim):
                return False
            return p == q

        if kind in ("floordiv", "ceildiv") and op.kind == "mul":
            if same(x, b) and isinstance(y, Dim):
                return y
            if same(y, b) and isinstance(x, Dim):
                return x
        if kind == "sub" and op.kind == "add":
            if same(y, b) and isinstance(x, Dim):
                return x
            if same(x, b) and isinstance(y, Dim):
                return y
        if kind == "add" and op.kind == "sub" and same(y, b) and isinstance(x, Dim):
            return x
        return None

    def __add__(self, other):
        if isinstance(other, int) and other == 0:
            return self
        return Dim._derive("add", [self, other])

    def __radd__(self, other):
        if isinstance(other, int) and other == 0:
            return self
        return Dim._derive("add", [other, self])

    def __sub__(self, other):
        if isinstance(other, int) and other == 0:
            return self
        return Dim._derive("sub", [self, other])

    def sub_left(self, other):
        """(-other) + self: removes from the left"""
        return Dim._derive("sub", [self, other], attribs={"left": True})

    def sub_right(self, other):
        """self - other"""
        return self - other

    def __mul__(self, other):
        if isinstance(other, int) and other == 1:
            return self
        return Dim._derive("mul", [self, other])

    def __rmul__(self, other):
        if isinstance(other, int) and other == 1:
            return self
        return Dim._derive("mul", [other, self])

    def __floordiv__(self, other):
        if isinstance(other, int) and other == 1:
            return self
        return Dim._derive("floordiv", [self, other])

    def div_left(self, other):
        """self // other where self = other * x"""
        return Dim._derive("floordiv", [self, other], attribs={"left": True})

    def div_right(self, other):
        """self // other"""
        return self // other

    def ceildiv_right(self, other):
        """ceil(self / other)"""
        if isinstance(other, int) and other == 1:
            return self
        return Dim._derive("ceildiv", [self, other])

    def ceildiv_left(self, other):
        """ceil(self / other)"""
        return Dim._derive("ceildiv", [self, other], attribs={"left": True})

    def __neg__(self):
        return Dim._derive("mul", [-1, self])

    def is_constant_static_dim(self) -> bool:
        """derived purely from constants"""
        return self.is_static()

    @property
    def description(self):
        """legacy alias for name"""
        return self.name

    @property
    def dyn_size_ext_raw(self):
        """raw sizes or None"""
        return self.dyn_size

    def get_vocab(self):
        """vocabulary or None"""
        return self.vocab


def _make_dim(dimension, name, kind, capacity, bounded_by, vocab):
    return Dim(dimension, name=name, kind=kind, capacity=capacity, bounded_by=bounded_by, vocab=vocab)


def _get_global_dim(name):
    return globals()[name]


batch_dim = Dim(None, name="batch", kind=DimTypes.Batch)
single_step_dim = Dim(1, name="single-step")
