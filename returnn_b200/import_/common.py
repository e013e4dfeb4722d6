"""
Package directory and module naming for :func:`returnn_b200.import_.import_`.

Every checkout becomes importable under the virtual package ``returnn_import``: the module for file ``a/b.py`` of repo
``github.com/u/r`` at version ``v`` is ``returnn_import.github_com.u.r.v<v>.a.b`` (``dev`` for the working tree).

Parity: returnn/import_/common.py (package_path :36, module_name :162).
"""

from __future__ import annotations
from typing import Optional
import importlib.util
import os
import re
import sys
import types

_EnvPkgPath = "RETURNN_PKG_PATH"
_DefaultPkgPath = "~/returnn/pkg"
ModuleNamePrefix = "returnn_import"


class InvalidVersion(Exception):
    """the version string does not have the form ``<date>-<commit>``"""


class MissingExplicitImport(ImportError):
    """a module of an imported repo was imported without going through :func:`import_` first"""


def package_path() -> str:
    """directory of all checkouts"""
    return os.path.abspath(os.path.expanduser(os.environ.get(_EnvPkgPath, _DefaultPkgPath)))


def _normalize(name: str) -> str:
    name = re.sub(r"[^A-Za-z0-9_]", "_", name)
    return ("_" + name) if name[:1].isdigit() else name


def _ensure_pkg(mod_name: str, path: Optional[str]):
    """register a namespace-like package module for ``mod_name`` (and its parents)"""
    parts = mod_name.split(".")
    for i in range(1, len(parts) + 1):
        name = ".".join(parts[:i])
        if name in sys.modules:
            continue
        mod = types.ModuleType(name)
        mod.__path__ = [path] if (i == len(parts) and path) else []
        mod.__package__ = name
        sys.modules[name] = mod
        if i > 1:
            setattr(sys.modules[".".join(parts[: i - 1])], parts[i - 1], mod)


def module_name(repo: str, repo_path: str, path: str, version: Optional[str], make_ready: bool = True) -> str:
    """
    :param repo: e.g. ``github.com/user/repo``
    :param repo_path: local checkout directory
    :param path: file or package directory inside the repo
    :param version: None = development working tree
    :param make_ready: register the parent packages in ``sys.modules`` so that ``importlib.import_module`` of the result works
    :return: dotted module name
    """
    full = os.path.join(repo_path, path)
    if not os.path.exists(full):
        raise ImportError("%s: %r does not exist in the checkout %s" % (repo, path, repo_path))
    rel = path[:-3] if path.endswith(".py") else path.rstrip("/")
    repo_mod = ".".join([ModuleNamePrefix] + [_normalize(p) for p in repo.split("/")] + ["v" + _normalize(version) if version else "dev"])
    name = repo_mod + "." + ".".join(_normalize(p) for p in rel.split("/"))
    if make_ready:
        _ensure_pkg(repo_mod, repo_path)
        # intermediate directories as packages with real paths so that relative imports inside the repo work
        cur_path, cur_name = repo_path, repo_mod
        for p in rel.split("/")[:-1]:
            cur_path = os.path.join(cur_path, p)
            cur_name = cur_name + "." + _normalize(p)
            _ensure_pkg(cur_name, cur_path)
        if name not in sys.modules:
            if os.path.isdir(full):
                init = os.path.join(full, "__init__.py")
                spec = importlib.util.spec_from_file_location(name, init if os.path.exists(init) else None, submodule_search_locations=[full])
                if spec is None or spec.loader is None:
                    _ensure_pkg(name, full)
                    return name
            else:
                spec = importlib.util.spec_from_file_location(name, full)
            mod = importlib.util.module_from_spec(spec)
            sys.modules[name] = mod
            try:
                spec.loader.exec_module(mod)
            except BaseException:
                sys.modules.pop(name, None)
                raise
            parent, _, leaf = name.rpartition(".")
            setattr(sys.modules[parent], leaf, mod)
    return name
