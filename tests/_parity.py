"""
Harness for tests that run the same model code against this framework and against the installed reference package
(``baseline/_ref``, importable as ``returnn``), in one process on the CPU.

A test case is written ONCE against an ``Api`` object (``api.rf``, ``api.Tensor``, ``api.Dim``, ``api.batch_dim``, ``api.bridge``)
and executed with both packages: the parameters of the reference module are copied into ours through the two ``state_dict``s
(so the keys and shapes must be identical), both get the same input arrays, and the outputs are compared.
The same cases are also run batched and one sequence at a time (padding invariance), without the reference.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple
import os
import sys
import types
import numpy
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF_DIR = os.path.join(_ROOT, "baseline", "_ref")
BEHAVIOR_VERSION = 24  # masks on by default in conv / pool / batch norm, "same" padding independent of the batch's longest sequence


class Api:
    """one of the two packages behind the same names"""

    def __init__(self, name: str, rf, Tensor, Dim, batch_dim, bridge, single_step_dim=None):
        self.name = name
        self.rf = rf
        self.Tensor = Tensor
        self.Dim = Dim
        self.batch_dim = batch_dim
        self.bridge = bridge
        self.single_step_dim = single_step_dim

    def setup(self):
        """
        Per-test state of this package: behaviour version and evaluation mode. Other tests of the suite run engines in this
        process and leave a global config, a train flag or another behaviour version behind.
        """
        import importlib

        basic = importlib.import_module(self.rf.__name__.rsplit(".", 1)[0] + (".utils.basic" if self.name == "ours" else ".util.basic"))
        if self.name == "ours":
            basic.BehaviorVersion._reset(BEHAVIOR_VERSION)
        else:
            basic.BehaviorVersion._reset()
            basic.BehaviorVersion.set(BEHAVIOR_VERSION)
        config_mod = importlib.import_module(self.rf.__name__.rsplit(".", 1)[0] + ".config")
        config_mod.set_global_config(None)
        self.rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)

    def mod(self, path: str):
        """submodule of the frontend package, e.g. ``"encoder.conformer"``"""
        import importlib

        return importlib.import_module(self.rf.__name__ + "." + path)

    def time_dim(self, lens: Sequence[int], name: str = "time"):
        """dynamic dim with per-sequence sizes"""
        # the batch dim gets its size too (some ops ask for it, e.g. when they build a mask from scratch)
        self.batch_dim.dyn_size_ext = self.Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(len(lens), dtype=torch.int32))
        d = self.Dim(None, name=name)
        d.dyn_size_ext = self.Tensor("%s_lens" % name, dims=[self.batch_dim], dtype="int32", raw_tensor=torch.tensor(list(lens), dtype=torch.int32))
        return d

    def tensor(self, name: str, dims, raw, *, dtype: Optional[str] = None, sparse_dim=None, feature_dim=None):
        """wrap a torch tensor / numpy array"""
        raw = torch.as_tensor(numpy.asarray(raw)) if not isinstance(raw, torch.Tensor) else raw
        if dtype is None:
            dtype = str(raw.dtype).replace("torch.", "")
        kwargs = {}
        if sparse_dim is not None:
            kwargs["sparse_dim"] = sparse_dim
        if feature_dim is not None:
            kwargs["feature_dim"] = feature_dim
        return self.Tensor(name, dims=list(dims), dtype=dtype, raw_tensor=raw.clone(), **kwargs)


_ours: Optional[Api] = None
_ref: Optional[Api] = None


def ours() -> Api:
    """this framework"""
    global _ours
    if _ours is None:
        import returnn_b200.frontend as rf
        from returnn_b200.tensor import Tensor, Dim, batch_dim, single_step_dim
        from returnn_b200.torch.frontend.bridge import rf_module_to_pt_module
        from returnn_b200.utils.basic import BehaviorVersion

        BehaviorVersion._reset(BEHAVIOR_VERSION)  # the same behaviour version as the reference side
        _ours = Api("ours", rf, Tensor, Dim, batch_dim, rf_module_to_pt_module, single_step_dim)
    return _ours


def reference_available() -> bool:
    """the reference package is installed in-tree"""
    return os.path.isdir(os.path.join(_REF_DIR, "returnn"))


def reference() -> Api:
    """the installed reference package (``import returnn``): never the alias of this framework"""
    global _ref
    if _ref is None:
        assert reference_available()
        mod = sys.modules.get("returnn")
        if mod is not None and not str(getattr(mod, "__file__", "")).startswith(_REF_DIR):
            raise RuntimeError("the name `returnn` is already taken by another module: %r" % getattr(mod, "__file__", None))
        if _REF_DIR not in sys.path:
            sys.path.insert(0, _REF_DIR)
        try:
            import tree  # noqa: F401
        except ImportError:
            sys.path.append(os.path.join(_ROOT, "baseline", "deps"))
        import returnn.frontend as rrf
        from returnn.tensor import Tensor, Dim, batch_dim, single_step_dim
        from returnn.torch.frontend.bridge import rf_module_to_pt_module
        from returnn.util.basic import BehaviorVersion

        BehaviorVersion._reset() if hasattr(BehaviorVersion, "_reset") else None
        BehaviorVersion.set(BEHAVIOR_VERSION)
        rrf.select_backend_torch()
        _ref = Api("reference", rrf, Tensor, Dim, batch_dim, rf_module_to_pt_module, single_step_dim)
    return _ref


def copy_params(src_api: Api, src_module, dst_api: Api, dst_module):
    """reference parameters -> our module, by state-dict name; keys and shapes must agree"""
    sd_src = src_api.bridge(src_module).state_dict()
    pt_dst = dst_api.bridge(dst_module)
    sd_dst = pt_dst.state_dict()
    assert sorted(sd_src.keys()) == sorted(sd_dst.keys()), "state-dict keys differ:\n  reference only: %s\n  ours only: %s" % (
        sorted(set(sd_src) - set(sd_dst)), sorted(set(sd_dst) - set(sd_src)))
    for k in sd_src:
        assert tuple(sd_src[k].shape) == tuple(sd_dst[k].shape), "shape of %r: reference %s, ours %s" % (k, tuple(sd_src[k].shape), tuple(sd_dst[k].shape))
    pt_dst.load_state_dict({k: v.detach().clone() for k, v in sd_src.items()})


def to_numpy_bt(api: Api, out, order: Sequence[Any]) -> numpy.ndarray:
    """raw values of ``out`` with the axes in the order of ``order`` (dims of ``out``)"""
    t = out.copy_transpose(list(order)) if hasattr(out, "copy_transpose") else out
    return t.raw_tensor.detach().cpu().float().numpy()


def masked(arr: numpy.ndarray, lens: Sequence[int], time_axis: int = 1) -> numpy.ndarray:
    """zero everything behind the sequence ends (batch axis 0)"""
    arr = arr.copy()
    for b, n in enumerate(lens):
        idx = [slice(None)] * arr.ndim
        idx[0] = b
        idx[time_axis] = slice(int(n), None)
        arr[tuple(idx)] = 0
    return arr


def assert_close(a: numpy.ndarray, b: numpy.ndarray, *, atol: float = 1e-5, rtol: float = 1e-4, what: str = ""):
    """shape and values"""
    assert a.shape == b.shape, "%s: shapes %s vs %s" % (what, a.shape, b.shape)
    err = numpy.abs(a - b)
    tol = atol + rtol * numpy.abs(b)
    assert (err <= tol).all(), "%s: max abs err %g (at %s), allowed %g" % (what, float(err.max()), numpy.unravel_index(err.argmax(), err.shape), float(tol.flat[err.argmax()]))
