"""
Git side of :func:`returnn_b200.import_.import_`: clone on first use, fetch when a revision is missing, one
``git worktree`` per pinned version.

Version format: ``<date>-<commit>`` with date ``YYYYMMDD[hh[mm[ss]]]`` and at least 7 hex digits of the commit; the
date must match the commit's committer date (a cheap guard against typos).

Parity: returnn/import_/git.py (stat_repo :59, get_repo_path :68).
"""

from __future__ import annotations
from typing import Optional
import os
import re
import subprocess
from . import common

_MinHashDigits = 7
_DateRe = re.compile(r"^\d{8}(\d{2}(\d{2}(\d{2})?)?)?$")
_RevRe = re.compile(r"^[0-9a-f]+$")
_RepoRe = re.compile(r"^[A-Za-z0-9_.\-]+(/[A-Za-z0-9_.\-]+)+$")


def _validate(repo: str, version: Optional[str]):
    if not _RepoRe.match(repo) or ".." in repo:
        raise ValueError("invalid repo %r (expected e.g. github.com/user/name)" % repo)
    if version is None:
        return
    if "-" not in version:
        raise common.InvalidVersion("version %r: expected <date>-<commit>" % version)
    date, rev = version.split("-", 1)
    if not _DateRe.match(date):
        raise common.InvalidVersion("version %r: invalid date %r" % (version, date))
    if not _RevRe.match(rev) or len(rev) < _MinHashDigits:
        raise common.InvalidVersion("version %r: commit needs >= %i hex digits" % (version, _MinHashDigits))


def _main_path(repo: str) -> str:
    return os.path.join(common.package_path(), repo)


def _version_path(repo: str, version: str) -> str:
    return "%s@v%s" % (_main_path(repo), version)


def _remote_url(repo: str) -> str:
    if repo.startswith("github.com/") or repo.startswith("gitlab.com/"):
        return "https://%s.git" % repo
    return "https://%s" % repo


def _git(args, cwd: Optional[str] = None) -> str:
    return subprocess.check_output(["git"] + list(args), cwd=cwd, stderr=subprocess.STDOUT).decode("utf8").strip()


def _ensure_main(repo: str) -> str:
    path = _main_path(repo)
    if not os.path.isdir(os.path.join(path, ".git")):
        os.makedirs(os.path.dirname(path), exist_ok=True)
        print("import_: git clone %s -> %s" % (_remote_url(repo), path))
        _git(["clone", _remote_url(repo), path])
    return path


def _has_rev(main: str, rev: str) -> bool:
    try:
        _git(["cat-file", "-e", rev + "^{commit}"], cwd=main)
        return True
    except subprocess.CalledProcessError:
        return False


def stat_repo(repo: str, version: Optional[str]):
    """make sure the checkout exists (clone / fetch / worktree)"""
    get_repo_path(repo, version)


def get_repo_path(repo: str, version: Optional[str], _report_dev_version_usage_stack_frame_depth: int = 1) -> str:
    """
    :return: local directory with the requested version checked out
    """
    _validate(repo, version)
    main = _ensure_main(repo)
    if version is None:
        print("import_: using the development working tree of %s (pin a version for reproducibility)" % repo)
        return main
    path = _version_path(repo, version)
    if os.path.isdir(path):
        return path
    date, rev = version.split("-", 1)
    if not _has_rev(main, rev):
        _git(["fetch", "--all"], cwd=main)
        if not _has_rev(main, rev):
            raise common.InvalidVersion("%s: commit %s not found" % (repo, rev))
    commit_date = _git(["show", "-s", "--format=%cd", "--date=format:%Y%m%d%H%M%S", rev], cwd=main)
    if not commit_date.startswith(date):
        raise common.InvalidVersion("%s: version %s has date %s but the commit is from %s" % (repo, version, date, commit_date))
    _git(["worktree", "add", "--detach", path, rev], cwd=main)
    return path
