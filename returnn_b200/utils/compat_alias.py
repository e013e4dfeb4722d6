"""
Import alias so that user configs written for RETURNN (``import returnn.frontend as rf``,
``from returnn.tensor import Dim``) load this package instead.

The mapping is by module path: ``returnn`` -> ``returnn_b200``, ``returnn.util`` -> ``returnn_b200.utils``.
The old flat module names (``import Config``, ``import TFUtil``; reference: returnn/__old_mod_loader__.py:1-228)
are covered for the modules that exist here.
"""

from __future__ import annotations
import importlib
import importlib.abc
import importlib.util
import sys

_SRC = "returnn"
_DST = "returnn_b200"

# old flat names -> new module path inside this package
_OLD_FLAT_NAMES = {
    "Config": "config",
    "Log": "log",
    "Util": "utils.basic",
    "Dataset": "datasets.basic",
    "GeneratingDataset": "datasets.generating",
    "HDFDataset": "datasets.hdf",
    "MetaDataset": "datasets.meta",
    "CachedDataset": "datasets.cached",
    "CachedDataset2": "datasets.cached2",
    "LearningRateControl": "learning_rate_control",
    "EngineBase": "engine.base",
    "EngineBatch": "engine.batch",
    "Pretrain": "pretrain",
    "Fsa": "utils.fsa",
    "Debug": "utils.debug",
    "NativeOp": "native_op",
}


def _translate(name: str) -> str:
    rest = name[len(_SRC) :]
    if rest == ".util" or rest.startswith(".util."):
        rest = ".utils" + rest[len(".util") :]
    return _DST + rest


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname == _SRC or fullname.startswith(_SRC + "."):
            tgt = _translate(fullname)
        elif fullname in _OLD_FLAT_NAMES:
            tgt = _DST + "." + _OLD_FLAT_NAMES[fullname]
        else:
            return None
        try:
            real = importlib.util.find_spec(tgt)
        except (ImportError, ValueError):
            real = None
        if real is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(tgt), is_package=real.submodule_search_locations is not None)
        return spec


_finder = None


def install(force: bool = False) -> bool:
    """
    Put the alias finder first on ``sys.meta_path``.

    :param force: drop an already imported foreign ``returnn`` package from ``sys.modules``
    :return: True if ``returnn`` now resolves to this package
    """
    global _finder
    existing = sys.modules.get(_SRC)
    if existing is not None and getattr(existing, "__name__", None) != _DST:
        if not force:
            return False
        for k in list(sys.modules):
            if k == _SRC or k.startswith(_SRC + "."):
                del sys.modules[k]
    if _finder is None:
        _finder = _AliasFinder()
        sys.meta_path.insert(0, _finder)
    return True


def uninstall():
    """Remove the alias finder and the aliased entries from ``sys.modules``."""
    global _finder
    if _finder is not None:
        try:
            sys.meta_path.remove(_finder)
        except ValueError:
            pass
        _finder = None
    for k in list(sys.modules):
        if k == _SRC or k.startswith(_SRC + "."):
            mod = sys.modules[k]
            if getattr(mod, "__name__", "").startswith(_DST):
                del sys.modules[k]
