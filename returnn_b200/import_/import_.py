"""
Parity: returnn/import_/import_.py:11.
"""

from __future__ import annotations
from typing import Optional
import importlib
from .git import get_repo_path
from .common import module_name


def import_(repo: str, path: str, version: Optional[str] = None):
    """
    :param repo: e.g. ``"github.com/rwth-i6/returnn-experiments"``
    :param path: file or package inside the repo, no leading slash
    :param version: ``"<date>-<commit>"``; None = the development working tree
    :return: the imported module
    """
    assert path and not path.startswith("/") and ".." not in path
    repo_path = get_repo_path(repo=repo, version=version)
    return importlib.import_module(module_name(repo=repo, repo_path=repo_path, path=path, version=version))
