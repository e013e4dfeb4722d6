"""
Import Python code from a Git repository by URL and pinned revision, for shareable experiment configs::

    from returnn_b200.import_ import import_
    mod = import_("github.com/rwth-i6/returnn-experiments", "common/models/transformer.py", "20211231-0123abcd0123")

Checkouts live under ``~/returnn/pkg`` (env ``RETURNN_PKG_PATH``): ``<repo>`` is the main clone (and the development
working tree used when ``version`` is None), ``<repo>@v<version>`` are ``git worktree`` checkouts that share its objects.

Parity: returnn/import_/ (import_.py:11, git.py, common.py).
"""

from .import_ import import_  # noqa: F401
from .common import package_path, module_name, InvalidVersion, MissingExplicitImport  # noqa: F401
