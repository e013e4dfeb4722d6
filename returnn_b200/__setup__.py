"""
Version string for packaging and for the startup banner: from ``git describe`` in a checkout, from ``_setup_info_generated``
in an installed package, else the static ``__version__``.

Parity: returnn/__setup__.py (get_version_str), setup.py.
"""

from __future__ import annotations
from typing import Optional
import os
import subprocess

_root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _git(args) -> Optional[str]:
    try:
        return subprocess.check_output(["git"] + list(args), cwd=_root, stderr=subprocess.DEVNULL).decode("utf8").strip()
    except (OSError, subprocess.CalledProcessError):
        return None


def get_version_str(verbose: bool = False, verbose_error: bool = False, fallback: Optional[str] = None, long: bool = False) -> str:
    """
    :param long: ``1.YYYYMMDD.HHMMSS+git.<rev>[.dirty]`` instead of ``1.YYYYMMDD.HHMMSS``
    :return: version derived from the date of the HEAD commit
    """
    try:
        from . import _setup_info_generated as info  # written by setup.py sdist/build

        return info.long_version if long else info.version
    except ImportError:
        pass
    if os.path.isdir(os.path.join(_root, ".git")):
        date = _git(["show", "-s", "--format=%cd", "--date=format:%Y%m%d.%H%M%S", "HEAD"])
        rev = _git(["rev-parse", "--short", "HEAD"])
        if date and rev:
            version = "1.%s" % date
            if long:
                dirty = _git(["status", "--porcelain", "--untracked-files=no"])
                version += "+git.%s%s" % (rev, ".dirty" if dirty else "")
            if verbose:
                print("version from git:", version)
            return version
        if verbose_error:
            print("git did not answer in", _root)
    if fallback is not None:
        return fallback
    from . import __version__, __long_version__

    return __long_version__ if long else __version__
