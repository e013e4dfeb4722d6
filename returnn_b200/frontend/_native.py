"""
Loader of the native dimension bookkeeping (``returnn_b200/csrc/pyext/rf_native.cpp``, built to ``ops/_build/_rf_native.so``).

:func:`setup` replaces the hot pure-Python helpers (``Tensor.get_out_permutation_to_dims``, ``Tensor.copy_compatible_to_dims_raw``,
``merge_dims_for_broadcast`` and the operand preparation of ``rf.combine`` / ``rf.compare``, i.e. of every ``a + b`` on tensors) by
versions that call the extension; the Python implementations stay as the fallback and as the specification. Controlled by the config option ``rf_native_opt`` /
environment ``RETURNN_B200_RF_NATIVE`` (default: on when the extension is built).

Parity: returnn/frontend/_native/__init__.py (get_module, setup).
"""

from __future__ import annotations
from typing import Optional
import importlib.util
import os

_mod = None
_tried = False
_is_set_up = False


def get_module(*, verbose: bool = False):
    """:return: the extension module or None"""
    global _mod, _tried
    if _tried:
        return _mod
    _tried = True
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ops", "_build", "_rf_native.so")
    if not os.path.exists(path):
        if verbose:
            print("rf native: %s not built" % path)
        return None
    try:
        spec = importlib.util.spec_from_file_location("_rf_native", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    except Exception as exc:  # wrong Python ABI etc.
        if verbose:
            print("rf native: cannot load %s: %s" % (path, exc))
        _mod = None
    return _mod


def setup(enable: Optional[bool] = None) -> bool:
    """install the native helpers; :return: whether they are active"""
    global _is_set_up
    if enable is None:
        enable = os.environ.get("RETURNN_B200_RF_NATIVE", "1") != "0"
    if not enable or _is_set_up:
        return _is_set_up
    mod = get_module()
    if mod is None:
        return False
    from ..tensor.tensor import Tensor
    from . import _utils, math_

    match_dims, merge_dims = mod.match_dims, mod.merge_dims

    def get_out_permutation_to_dims(self, dims):
        """perm such that copy_transpose(perm).dims == dims (native matching)"""
        own = self._dims
        assert len(dims) == len(own), "%r: cannot permute to %r" % (self, dims)
        perm = match_dims(own, dims)
        if -1 in perm:
            raise ValueError("%r: dim %r not found for permutation to %r" % (self, dims[perm.index(-1)], dims))
        return perm

    def merge_dims_for_broadcast(a, b):
        """dims of a binary op's result (native)"""
        return merge_dims(a._dims, b._dims)

    if hasattr(mod, "bin_op_prepare"):
        copy_compatible_raw, bin_op_prepare = mod.copy_compatible_raw, mod.bin_op_prepare
        py_copy_compatible = Tensor.copy_compatible_to_dims_raw

        def copy_compatible_to_dims_raw(self, dims, *, unbroadcast: bool = False):
            """raw tensor with axes in the order of ``dims`` (native); the broadcasting form stays in Python"""
            if unbroadcast or not hasattr(self._raw_tensor, "permute"):
                return py_copy_compatible(self, dims, unbroadcast=unbroadcast)
            return copy_compatible_raw(self._raw_tensor, self._dims, dims)

        py_prep_bin = math_._prep_bin

        def _prep_bin(a, b, allow_broadcast_all_sources, dim_order):
            """operands of a binary op as raw views over the merged dims (native when both are Tensors and nothing special is asked)"""
            if type(a) is Tensor and type(b) is Tensor and allow_broadcast_all_sources is not False and dim_order is None:
                ra, rb, out_dims = bin_op_prepare(a._raw_tensor, a._dims, b._raw_tensor, b._dims)
                return a, b, ra, rb, out_dims
            return py_prep_bin(a, b, allow_broadcast_all_sources, dim_order)

        Tensor.copy_compatible_to_dims_raw = copy_compatible_to_dims_raw
        math_._prep_bin = _prep_bin
    Tensor.get_out_permutation_to_dims = get_out_permutation_to_dims
    _utils.merge_dims_for_broadcast = merge_dims_for_broadcast
    if hasattr(math_, "merge_dims_for_broadcast"):
        math_.merge_dims_for_broadcast = merge_dims_for_broadcast
    _is_set_up = True
    return True
