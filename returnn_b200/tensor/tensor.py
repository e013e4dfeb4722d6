"""
``Tensor``: a raw ``torch.Tensor`` (or numpy array) plus named dims, dtype string, optional sparse/feature dim.

All RF functions take and return ``Tensor``. Axis matching between tensors is by ``Dim`` identity, never by position.

Parity: returnn/tensor/tensor.py:39, returnn/tensor/_tensor_extra.py (copy_* family, masks, axis lookup),
returnn/tensor/_tensor_op_overloads.py.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union
import numpy
from .dim import Dim, batch_dim, single_step_dim, DimTypes, VerifyOutShapeException
from ..utils.basic import NotSpecified

__all__ = ["Tensor"]

_float_dtypes = ("float16", "bfloat16", "float32", "float64")
_int_dtypes = ("int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64")


def _raw_dtype_str(raw) -> str:
    import torch

    if isinstance(raw, torch.Tensor):
        return str(raw.dtype).split(".")[-1]
    dt = numpy.asarray(raw).dtype
    if dt.kind in "US":
        return "string"
    return str(dt)


class Tensor:
    """
    Named-dimension tensor.
    """

    __slots__ = (
        "name",
        "_dims",
        "dtype",
        "sparse_dim",
        "_feature_dim",
        "_raw_tensor",
        "version",
        "control_flow_ctx",
        "available_for_inference",
        "_extra",
    )
    size_dtype = "int32"

    def __init__(
        self,
        name: str,
        dims: Sequence[Dim],
        dtype: Optional[str] = None,
        *,
        sparse_dim: Optional[Dim] = None,
        feature_dim: Optional[Dim] = NotSpecified,
        feature_dim_axis=NotSpecified,
        raw_tensor=None,
        version: int = 2,
        available_for_inference: bool = True,
        control_flow_ctx=None,
        **kwargs,
    ):
        """
        :param name: for humans
        :param dims: one Dim per axis of raw_tensor, in order
        :param dtype: e.g. "float32", "bfloat16", "int32", "bool". Default float32, or int32 if sparse.
        :param sparse_dim: the values are class indices into this dim
        :param feature_dim: NotSpecified: the last static non-batch dim for dense float tensors
        :param raw_tensor: torch.Tensor / numpy array / None (template)
        """
        assert isinstance(name, str), "Tensor name must be str, got %r" % (name,)
        dims = tuple(dims)
        for d in dims:
            assert isinstance(d, Dim), "Tensor %r: dims must be Dim objects, got %r" % (name, d)
        if kwargs:
            kwargs.pop("time_dim_axis", None)
            kwargs.pop("batch", None)
            kwargs.pop("beam", None)
            kwargs.pop("vocab", None)
            if "dim" in kwargs or "shape" in kwargs:
                raise TypeError("Tensor %r: legacy shape/dim kwargs are not supported; give dims=[...]" % name)
            kwargs.pop("placeholder", None)
            assert not kwargs, "Tensor %r: unexpected kwargs %r" % (name, kwargs)
        self.name = name
        self._dims = dims
        if dtype is None:
            dtype = "int32" if sparse_dim is not None else "float32"
        self.dtype = dtype
        self.sparse_dim = sparse_dim
        if feature_dim is NotSpecified and feature_dim_axis is not NotSpecified and feature_dim_axis is not None:
            feature_dim = dims[feature_dim_axis]
        self._feature_dim = feature_dim
        self.version = version
        self.control_flow_ctx = control_flow_ctx
        self.available_for_inference = available_for_inference
        self._extra = None
        self._raw_tensor = None
        if raw_tensor is not None:
            self.raw_tensor = raw_tensor

    # -- basic properties --------------------------------------------------------------------------
    @property
    def dims(self) -> Tuple[Dim, ...]:
        """dims in raw order"""
        return self._dims

    @property
    def dim_tags(self) -> Tuple[Dim, ...]:
        """legacy alias"""
        return self._dims

    @property
    def dims_set(self):
        """set of dims"""
        return set(self._dims)

    @property
    def batch_ndim(self) -> int:
        """number of axes"""
        return len(self._dims)

    ndim = batch_ndim

    @property
    def raw_tensor(self):
        """the framework tensor"""
        return self._raw_tensor

    @raw_tensor.setter
    def raw_tensor(self, value):
        if value is not None:
            shape = tuple(value.shape)
            if len(shape) != len(self._dims):
                raise ValueError(
                    "%r: raw tensor ndim %i != len(dims) %i (shape %r)" % (self, len(shape), len(self._dims), shape)
                )
            for i, d in enumerate(self._dims):
                if d.dimension is not None and shape[i] != d.dimension:
                    raise ValueError("%r: raw tensor shape %r does not match dims at axis %i" % (self, shape, i))
            rd = _raw_dtype_str(value)
            if rd != self.dtype:
                raise ValueError("%r: raw tensor dtype %s != %s" % (self, rd, self.dtype))
        self._raw_tensor = value

    placeholder = raw_tensor

    @property
    def feature_dim(self) -> Optional[Dim]:
        """feature dim (explicit, or the last static non-batch dim of a dense float tensor)"""
        if self._feature_dim is not NotSpecified:
            return self._feature_dim
        if self.sparse_dim is not None or self.dtype not in _float_dtypes:
            return None
        for d in reversed(self._dims):
            if d.is_static() and not d.is_batch_dim() and d.kind is not DimTypes.Spatial:
                return d
        return None

    @feature_dim.setter
    def feature_dim(self, value: Optional[Dim]):
        assert value is None or value in self._dims
        self._feature_dim = value

    @property
    def feature_dim_axis(self) -> Optional[int]:
        """axis of the feature dim"""
        fd = self.feature_dim
        return None if fd is None else self._dims.index(fd)

    @property
    def sparse(self) -> bool:
        """class indices"""
        return self.sparse_dim is not None

    @property
    def dim(self) -> Optional[int]:
        """number of classes if sparse, else feature dimension"""
        if self.sparse_dim is not None:
            return self.sparse_dim.dimension
        fd = self.feature_dim
        return None if fd is None else fd.dimension

    @property
    def device(self) -> Optional[str]:
        """device of raw tensor as str"""
        if self._raw_tensor is None:
            return None
        dev = getattr(self._raw_tensor, "device", None)
        return None if dev is None else str(dev)

    @property
    def shape(self) -> Tuple[Optional[int], ...]:
        """static sizes without the batch dim, None for dynamic dims"""
        return tuple(d.dimension for d in self._dims if not d.is_batch_dim())

    @property
    def batch_shape(self) -> Tuple[Optional[int], ...]:
        """static sizes with batch, None for dynamic"""
        return tuple(d.dimension for d in self._dims)

    def have_batch_axis(self) -> bool:
        """batch_dim in dims"""
        return any(d.is_batch_dim() for d in self._dims)

    def have_time_axis(self) -> bool:
        """a time (first dynamic / spatial) axis exists"""
        return self.time_dim_axis is not None

    def have_feature_axis(self) -> bool:
        """feature dim exists"""
        return self.feature_dim is not None

    @property
    def batch_dim_axis(self) -> Optional[int]:
        """axis of batch dim"""
        for i, d in enumerate(self._dims):
            if d.is_batch_dim():
                return i
        return None

    @property
    def time_dim_axis(self) -> Optional[int]:
        """first dynamic (or spatial) non-batch axis"""
        for i, d in enumerate(self._dims):
            if not d.is_batch_dim() and (d.is_dynamic() or d.kind is DimTypes.Spatial):
                return i
        return None

    def get_time_dim_tag(self) -> Dim:
        """the time dim"""
        ax = self.time_dim_axis
        assert ax is not None, "%r has no time axis" % self
        return self._dims[ax]

    def is_float(self) -> bool:
        """float dtype"""
        return self.dtype in _float_dtypes

    def is_int(self) -> bool:
        """int dtype"""
        return self.dtype in _int_dtypes

    def __repr__(self):
        return "Tensor{%r, [%s]%s%s}" % (
            self.name,
            ",".join(d.short_repr() for d in self._dims),
            ", dtype=%r" % self.dtype if self.dtype != "float32" else "",
            ", sparse_dim=%r" % self.sparse_dim if self.sparse_dim is not None else "",
        )

    def __bool__(self):
        if self._raw_tensor is None or self._dims:
            raise ValueError("%r: truth value is ambiguous (only scalars with a value can be used as bool)" % self)
        return bool(self._raw_tensor)

    def __hash__(self):
        return id(self)

    def __getstate__(self):
        d = {k: getattr(self, k) for k in self.__slots__ if k not in ("_raw_tensor", "_extra", "control_flow_ctx")}
        raw = self._raw_tensor
        if raw is not None and not isinstance(raw, numpy.ndarray):
            raw = raw.detach().cpu()
        d["_raw_tensor"] = raw
        return d

    def __setstate__(self, state):
        for k in self.__slots__:
            object.__setattr__(self, k, state.get(k, None))

    def get_kwargs(self, *, include_special_axes=True) -> Dict[str, Any]:
        """kwargs to recreate the template"""
        kw: Dict[str, Any] = {"name": self.name, "dims": self._dims, "dtype": self.dtype}
        if self.sparse_dim is not None:
            kw["sparse_dim"] = self.sparse_dim
        if self._feature_dim is not NotSpecified:
            kw["feature_dim"] = self._feature_dim
        if not self.available_for_inference:
            kw["available_for_inference"] = False
        return kw

    # -- copies ------------------------------------------------------------------------------------
    def copy(self, name: Optional[str] = None) -> "Tensor":
        """shallow copy (same raw tensor)"""
        t = Tensor(**self.get_kwargs())
        if name:
            t.name = name
        t._raw_tensor = self._raw_tensor
        t.control_flow_ctx = self.control_flow_ctx
        return t

    def copy_template(self, name: Optional[str] = None, *, dtype: Optional[str] = None) -> "Tensor":
        """copy without raw tensor"""
        kw = self.get_kwargs()
        if name:
            kw["name"] = name
        if dtype:
            kw["dtype"] = dtype
        return Tensor(**kw)

    def copy_with_raw(self, raw) -> "Tensor":
        """same meta, other raw tensor"""
        t = Tensor(**self.get_kwargs())
        t._raw_tensor = raw
        return t

    def copy_template_new_dim_tags(self, new_dim_tags: Sequence[Dim], name: Optional[str] = None, keep_special_axes: bool = False) -> "Tensor":
        """template with other dims"""
        kw = self.get_kwargs()
        old = self._dims
        kw["dims"] = tuple(new_dim_tags)
        if keep_special_axes and self._feature_dim is not NotSpecified and self._feature_dim is not None:
            kw["feature_dim"] = new_dim_tags[old.index(self._feature_dim)]
        elif self._feature_dim is not NotSpecified and self._feature_dim not in new_dim_tags:
            kw.pop("feature_dim", None)
        if name:
            kw["name"] = name
        return Tensor(**kw)

    def copy_template_replace_dim_tag(self, axis: int, new_dim_tag: Dim, name: Optional[str] = None) -> "Tensor":
        """template with dims[axis] replaced"""
        dims = list(self._dims)
        old = dims[axis]
        dims[axis] = new_dim_tag
        kw = self.get_kwargs()
        kw["dims"] = tuple(dims)
        if self._feature_dim is not NotSpecified and self._feature_dim == old:
            kw["feature_dim"] = new_dim_tag
        if name:
            kw["name"] = name
        return Tensor(**kw)

    def copy_template_excluding_axis(self, exclude_axis: int, name: Optional[str] = None) -> "Tensor":
        """template without one axis"""
        dims = list(self._dims)
        removed = dims.pop(exclude_axis)
        kw = self.get_kwargs()
        kw["dims"] = tuple(dims)
        if kw.get("feature_dim", None) == removed:
            kw.pop("feature_dim")
        if name:
            kw["name"] = name
        return Tensor(**kw)

    def copy_template_adding_time_dim(self, name=None, time_dim_axis=0) -> "Tensor":
        """template with a new dynamic time dim"""
        dims = list(self._dims)
        dims.insert(time_dim_axis, Dim(None, name="time", kind=DimTypes.Spatial))
        kw = self.get_kwargs()
        kw["dims"] = tuple(dims)
        if name:
            kw["name"] = name
        return Tensor(**kw)

    def copy_transpose(self, perm: Sequence[int]) -> "Tensor":
        """permute axes"""
        perm = [self.get_axis_from_description(a) if isinstance(a, Dim) else int(a) for a in perm]
        assert sorted(perm) == list(range(len(self._dims)))
        if perm == list(range(len(self._dims))):
            return self.copy()
        kw = self.get_kwargs()
        kw["dims"] = tuple(self._dims[i] for i in perm)
        t = Tensor(**kw)
        if self._raw_tensor is not None:
            raw = self._raw_tensor
            t._raw_tensor = raw.permute(*perm) if hasattr(raw, "permute") else raw.transpose(perm)
        return t

    def copy_transpose_to_dims(self, dims: Sequence[Dim]) -> "Tensor":
        """permute axes to the given order"""
        return self.copy_transpose(self.get_out_permutation_to_dims(dims))

    def get_out_permutation_to_dims(self, dims: Sequence[Dim]) -> List[int]:
        """perm such that copy_transpose(perm).dims == dims"""
        assert len(dims) == len(self._dims), "%r: cannot permute to %r" % (self, dims)
        rem = list(range(len(self._dims)))
        perm = []
        for d in dims:
            found = None
            for i in rem:
                if self._dims[i] == d:
                    found = i
                    break
            if found is None:
                raise ValueError("%r: dim %r not found for permutation to %r" % (self, d, dims))
            rem.remove(found)
            perm.append(found)
        return perm

    def copy_move_axis(self, old_axis: int, new_axis: int) -> "Tensor":
        """move one axis"""
        n = len(self._dims)
        if old_axis < 0:
            old_axis += n
        if new_axis < 0:
            new_axis += n
        perm = list(range(n))
        perm.pop(old_axis)
        perm.insert(new_axis, old_axis)
        return self.copy_transpose(perm)

    def copy_as_batch_major(self) -> "Tensor":
        """batch first"""
        ax = self.batch_dim_axis
        assert ax is not None
        return self.copy_move_axis(ax, 0)

    def copy_as_time_major(self) -> "Tensor":
        """time first"""
        ax = self.time_dim_axis
        assert ax is not None
        return self.copy_move_axis(ax, 0)

    def copy_with_feature_last(self) -> "Tensor":
        """feature last"""
        ax = self.feature_dim_axis
        assert ax is not None
        return self.copy_move_axis(ax, -1)

    def copy_with_feature_dim_axis(self, feature_dim_axis: int) -> "Tensor":
        """feature at axis"""
        ax = self.feature_dim_axis
        assert ax is not None
        return self.copy_move_axis(ax, feature_dim_axis)

    def copy_add_dim_by_tag(self, dim_tag: Dim, unbroadcast: bool = False, axis: Optional[int] = None) -> "Tensor":
        """insert an axis of size 1 (or expanded when unbroadcast)"""
        if axis is None:
            axis = len(self._dims)
        if axis < 0:
            axis += len(self._dims) + 1
        dims = list(self._dims)
        dims.insert(axis, dim_tag)
        kw = self.get_kwargs()
        kw["dims"] = tuple(dims)
        t = Tensor(**kw)
        if self._raw_tensor is not None:
            raw = self._raw_tensor.unsqueeze(axis) if hasattr(self._raw_tensor, "unsqueeze") else numpy.expand_dims(self._raw_tensor, axis)
            if unbroadcast or dim_tag.dimension not in (None, 1):
                size = dim_tag.get_dim_value()
                shape = list(raw.shape)
                shape[axis] = size
                raw = raw.expand(*shape) if hasattr(raw, "expand") else numpy.broadcast_to(raw, shape)
            elif dim_tag.dimension is None:
                # dynamic dim, broadcast with size 1 is not a valid raw shape for this dim -> expand
                size = dim_tag.get_dim_value()
                shape = list(raw.shape)
                shape[axis] = size
                raw = raw.expand(*shape) if hasattr(raw, "expand") else numpy.broadcast_to(raw, shape)
            t._raw_tensor = raw
        return t

    def copy_compatible_to_dims(self, dims: Sequence[Dim], *, unbroadcast: bool = False) -> "Tensor":
        """
        Permute and add broadcast axes so that the result has exactly ``dims``.
        Missing dims become size-1 axes unless ``unbroadcast``.
        """
        raw = self.copy_compatible_to_dims_raw(dims, unbroadcast=unbroadcast) if self._raw_tensor is not None else None
        kw = self.get_kwargs()
        kw["dims"] = tuple(dims)
        t = Tensor(**kw)
        t._raw_tensor = raw  # broadcast axes have raw size 1: bypass the shape check
        return t

    def copy_compatible_to_dims_raw(self, dims: Sequence[Dim], *, unbroadcast: bool = False):
        """
        :return: raw tensor with axes in the order of ``dims``; dims that self lacks have size 1
        """
        raw = self._raw_tensor
        assert raw is not None, "%r: no raw tensor" % self
        own = self._dims
        n_own = len(own)
        if n_own == len(dims):
            same = True
            for a, b in zip(own, dims):
                if a is not b and a != b:
                    same = False
                    break
            if same:
                return raw
        used = [False] * n_own
        perm: List[int] = []
        out_is_new: List[bool] = []
        for d in dims:
            found = -1
            for i in range(n_own):
                if not used[i] and (own[i] is d or own[i] == d):
                    found = i
                    break
            if found >= 0:
                used[found] = True
                perm.append(found)
                out_is_new.append(False)
            else:
                out_is_new.append(True)
        if not all(used):
            missing = [own[i] for i in range(n_own) if not used[i]]
            raise ValueError("%r: dims %r not in target dims %r" % (self, missing, list(dims)))
        is_torch = hasattr(raw, "permute")
        if perm != sorted(perm):
            raw = raw.permute(*perm) if is_torch else raw.transpose(perm)
        if len(dims) != n_own:
            shape = []
            it = iter(raw.shape)
            for new in out_is_new:
                shape.append(1 if new else next(it))
            raw = raw.reshape(shape) if not is_torch else raw.reshape(shape)
        if unbroadcast and any(out_is_new):
            shape = [d.get_dim_value() if new else s for d, new, s in zip(dims, out_is_new, raw.shape)]
            raw = raw.expand(*shape) if is_torch else numpy.broadcast_to(raw, shape)
        return raw

    def copy_compatible_to(self, other: "Tensor", *, unbroadcast: bool = False, **_kwargs) -> "Tensor":
        """like copy_compatible_to_dims(other.dims)"""
        return self.copy_compatible_to_dims(other.dims, unbroadcast=unbroadcast)

    def num_elements(self):
        """number of (non-padded) elements: an int, or a scalar Tensor when sequence lengths live on the device"""
        from .. import frontend as rf

        return rf.num_elements_of_shape(self.dims)

    def copy_masked(self, mask_value, *, dims: Optional[Sequence[Dim]] = None, allow_int=NotSpecified) -> "Tensor":
        """padded frames of all dynamic dims (or given dims) set to mask_value"""
        from .. import frontend as rf

        res = self
        for d in dims if dims is not None else self._dims:
            if d.is_batch_dim() or not d.need_masking() or d.dyn_size_ext is None:
                continue
            if not d.is_dynamic_seq_length():
                continue
            mask = d.get_mask(device=self.device)
            res = rf.where(mask, res, mask_value)
        return res

    def copy_squeeze_axes(self, axes: Sequence[int]) -> "Tensor":
        """remove size-1 axes"""
        axes = sorted(axes, reverse=True)
        t = self
        for a in axes:
            assert t._dims[a].dimension == 1
            tpl = t.copy_template_excluding_axis(a)
            if t._raw_tensor is not None:
                tpl._raw_tensor = t._raw_tensor.squeeze(a)
            t = tpl
        return t

    # -- axes lookup -------------------------------------------------------------------------------
    def get_axis_from_description(self, axis, allow_int: bool = True) -> int:
        """Dim / int / 'B' / 'T' / 'F' -> axis index"""
        axes = self.get_axes_from_description(axis, allow_int=allow_int)
        assert len(axes) == 1, "%r: %r is not a unique axis (got %r)" % (self, axis, axes)
        return axes[0]

    def get_axes_from_description(self, axes, allow_int: bool = True) -> List[int]:
        """Dim / int / str / list of those -> axis indices"""
        if axes is None:
            return []
        if isinstance(axes, Dim):
            return [i for i, d in enumerate(self._dims) if d == axes]
        if isinstance(axes, int):
            assert allow_int
            return [axes % len(self._dims)]
        if isinstance(axes, str):
            s = axes.lower()
            if s in ("b", "batch"):
                return [self.batch_dim_axis] if self.batch_dim_axis is not None else []
            if s in ("t", "time"):
                return [self.time_dim_axis] if self.time_dim_axis is not None else []
            if s in ("f", "feature"):
                return [self.feature_dim_axis] if self.feature_dim_axis is not None else []
            if s in ("*", "all"):
                return list(range(len(self._dims)))
            if s == "spatial":
                return [i for i, d in enumerate(self._dims) if not d.is_batch_dim() and d != self.feature_dim]
            raise ValueError("%r: invalid axis description %r" % (self, axes))
        res = []
        for a in axes:
            for i in self.get_axes_from_description(a, allow_int=allow_int):
                if i not in res:
                    res.append(i)
        return res

    def get_dim_tag(self, axis: int) -> Dim:
        """dims[axis]"""
        return self._dims[axis]

    def get_dim_tag_from_description(self, axis) -> Dim:
        """Dim by description"""
        return self._dims[self.get_axis_from_description(axis)]

    def get_batch_shape(self, batch_dim) -> Tuple[Optional[int], ...]:
        """shape with batch replaced"""
        return tuple(batch_dim if d.is_batch_dim() else d.dimension for d in self._dims)

    def get_dynamic_axes(self) -> List[int]:
        """axes with dynamic non-batch dims"""
        return [i for i, d in enumerate(self._dims) if d.is_dynamic() and not d.is_batch_dim()]

    def get_static_axes(self) -> List[int]:
        """axes with static dims"""
        return [i for i, d in enumerate(self._dims) if d.is_static()]

    def get_sequence_lengths(self):
        """raw seq lens of the time dim"""
        return self.get_time_dim_tag().dyn_size

    def get_sequence_mask_broadcast(self, axis=None) -> Any:
        """raw bool mask broadcastable to self"""
        if axis is None:
            axis = self.time_dim_axis
        d = self._dims[self.get_axis_from_description(axis)]
        return d.get_mask(device=self.device).copy_compatible_to_dims_raw(self._dims)

    def get_sequence_mask_tensor(self, axis: int) -> "Tensor":
        """mask Tensor of dims[axis]"""
        return self._dims[axis].get_mask(device=self.device)

    def mark_same_time(self, tags, must_match=False) -> bool:
        """legacy: no-op"""
        return False

    def verify_out_shape(self, out_shape, allow_missing_implicit_dims: bool = False):
        """check dims as a set"""
        if out_shape is None:
            return
        expected = set(out_shape)
        have = set(self._dims)
        if expected != have:
            raise VerifyOutShapeException("%r verify_out_shape: expected %r, have %r" % (self, expected, have))

    def sanity_check(self, ignore_placeholder=False, assume_complete=True):
        """consistency"""
        if self._feature_dim is not NotSpecified and self._feature_dim is not None:
            assert self._feature_dim in self._dims
        if self.sparse_dim is not None:
            assert self.dtype in _int_dtypes, "%r: sparse but dtype %s" % (self, self.dtype)

    # -- run ctx shortcuts -------------------------------------------------------------------------
    def mark_as_loss(self, name: str, *, scale: Optional[float] = 1.0, as_error: bool = False,
                     use_normalized_loss: bool = False, use_flatten_frames: bool = True,
                     custom_inv_norm_factor: Optional["Tensor"] = None) -> None:
        """register as loss in the current run ctx"""
        from .. import frontend as rf

        rf.get_run_ctx().mark_as_loss(
            loss=self, name=name, scale=scale, as_error=as_error, use_normalized_loss=use_normalized_loss,
            use_flatten_frames=use_flatten_frames, custom_inv_norm_factor=custom_inv_norm_factor)

    def mark_as_output(self, name: str, *, shape: Optional[Sequence[Dim]] = None) -> None:
        """register as output in the current run ctx"""
        from .. import frontend as rf

        rf.get_run_ctx().mark_as_output(self, name=name, dims=shape)

    def mark_as_default_output(self, *, shape: Optional[Sequence[Dim]] = None) -> None:
        """register as the output named "output" """
        from .. import frontend as rf

        rf.get_run_ctx().mark_as_default_output(self, shape=shape)

    # -- operators ---------------------------------------------------------------------------------
    def _rf(self):
        from .. import frontend as rf

        return rf

    def __eq__(self, other):
        if self._raw_tensor is None:
            return self is other
        return self._rf().compare(self, "==", other)

    def __ne__(self, other):
        if self._raw_tensor is None:
            return self is not other
        return self._rf().compare(self, "!=", other)

    def __lt__(self, other):
        return self._rf().compare(self, "<", other)

    def __le__(self, other):
        return self._rf().compare(self, "<=", other)

    def __gt__(self, other):
        return self._rf().compare(self, ">", other)

    def __ge__(self, other):
        return self._rf().compare(self, ">=", other)

    def __add__(self, other):
        return self._rf().combine(self, "+", other)

    def __radd__(self, other):
        return self._rf().combine(other, "+", self)

    def __sub__(self, other):
        return self._rf().combine(self, "-", other)

    def __rsub__(self, other):
        return self._rf().combine(other, "-", self)

    def __mul__(self, other):
        return self._rf().combine(self, "*", other)

    def __rmul__(self, other):
        return self._rf().combine(other, "*", self)

    def __truediv__(self, other):
        return self._rf().combine(self, "/", other)

    def __rtruediv__(self, other):
        return self._rf().combine(other, "/", self)

    def __floordiv__(self, other):
        return self._rf().combine(self, "//", other)

    def __rfloordiv__(self, other):
        return self._rf().combine(other, "//", self)

    def __mod__(self, other):
        return self._rf().combine(self, "%", other)

    def __rmod__(self, other):
        return self._rf().combine(other, "%", self)

    def __pow__(self, other):
        return self._rf().combine(self, "**", other)

    def __rpow__(self, other):
        return self._rf().combine(other, "**", self)

    def __neg__(self):
        return self._rf().neg(self)

    def __invert__(self):
        return self._rf().logical_not(self)

    def __abs__(self):
        return self._rf().abs(self)

    def __ceil__(self):
        return self._rf().ceil(self)

    def __floor__(self):
        return self._rf().floor(self)

    def __and__(self, other):
        return self._rf().combine(self, "logical_and", other)

    def __rand__(self, other):
        return self._rf().combine(other, "logical_and", self)

    def __or__(self, other):
        return self._rf().combine(self, "logical_or", other)

    def __ror__(self, other):
        return self._rf().combine(other, "logical_or", self)

    def __matmul__(self, other):
        raise TypeError("use rf.matmul(a, b, reduce=dim): named dims need the reduce dim to be explicit")
