"""
Local file cache: copies remote (NFS) files to a local cache directory, keyed by path, with size and mtime checks,
lock files so that several processes copy a file only once, keep-alive touching of files in use and cleanup of stale
files when space is needed.

Parity: returnn/util/file_cache.py:1-656 (FileCache.get_file, handle_cached_files_in_config, CachedFile).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Tuple
import os
import shutil
import threading
import time
from .basic import LockFile, get_temp_dir

__all__ = ["FileCache", "CachedFile", "get_instance", "get_instance_if_enabled", "handle_cached_files_in_config"]


class CachedFile:
    """marks a config entry as "copy through the file cache before use" """

    def __init__(self, filename: str):
        self.filename = filename

    def __repr__(self):
        return "CachedFile(%r)" % self.filename


class FileCache:
    """the cache"""

    def __init__(self, *, cache_directory: Optional[str] = None, cleanup_files_always_older_than_days: float = 31.0,
                 cleanup_files_wanted_older_than_days: float = 1.0, cleanup_disk_usage_wanted_free_ratio: float = 0.2,
                 num_tries: int = 3):
        if cache_directory is None:
            cache_directory = os.path.join(get_temp_dir(), "returnn_b200", "file_cache")
        self.cache_directory = os.path.expanduser(cache_directory)
        self._always_older = cleanup_files_always_older_than_days * 86400
        self._wanted_older = cleanup_files_wanted_older_than_days * 86400
        self._wanted_free_ratio = cleanup_disk_usage_wanted_free_ratio
        self._num_tries = num_tries
        self._in_use: Dict[str, int] = {}
        self._lock = threading.Lock()
        self._touch_thread: Optional[threading.Thread] = None
        self._stop = threading.Event()

    def _dst(self, src: str) -> str:
        return os.path.join(self.cache_directory, os.path.abspath(src).lstrip("/"))

    def get_file(self, src_filename: str) -> str:
        """:return: local path with the same content; the file is marked in use until release_files"""
        dst = self._dst(src_filename)
        last_exc = None
        for _ in range(self._num_tries):
            try:
                self._copy_if_needed(src_filename, dst)
                break
            except OSError as exc:
                last_exc = exc
                time.sleep(1)
        else:
            raise last_exc
        with self._lock:
            self._in_use[dst] = self._in_use.get(dst, 0) + 1
            if self._touch_thread is None:
                self._touch_thread = threading.Thread(target=self._touch_loop, name="FileCache-keepalive", daemon=True)
                self._touch_thread.start()
        return dst

    def release_files(self, filenames):
        """not in use anymore"""
        if isinstance(filenames, str):
            filenames = [filenames]
        with self._lock:
            for fn in filenames:
                if fn in self._in_use:
                    self._in_use[fn] -= 1
                    if self._in_use[fn] <= 0:
                        del self._in_use[fn]

    def _is_up_to_date(self, src: str, dst: str) -> bool:
        try:
            s, d = os.stat(src), os.stat(dst)
        except OSError:
            return False
        return s.st_size == d.st_size and d.st_mtime >= s.st_mtime

    def _copy_if_needed(self, src: str, dst: str):
        if self._is_up_to_date(src, dst):
            os.utime(dst, None)
            return
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        with LockFile(os.path.dirname(dst), name=os.path.basename(dst) + ".lock"):
            if self._is_up_to_date(src, dst):
                return
            size = os.stat(src).st_size
            self.cleanup(need_at_least_free_space_size=size)
            tmp = dst + ".copy"
            shutil.copyfile(src, tmp)
            os.replace(tmp, dst)
            os.utime(dst, None)

    def _touch_loop(self):
        while not self._stop.wait(60.0):
            with self._lock:
                files = list(self._in_use)
            for fn in files:
                try:
                    os.utime(fn, None)
                except OSError:
                    pass

    def cleanup(self, *, need_at_least_free_space_size: int = 0):
        """delete stale files: always those older than the hard limit; older than the soft limit only if space is short"""
        if not os.path.isdir(self.cache_directory):
            return
        now = time.time()
        usage = shutil.disk_usage(self.cache_directory)
        want_free = max(need_at_least_free_space_size, int(self._wanted_free_ratio * usage.total))
        entries: List[Tuple[float, str, int]] = []
        for root, _, files in os.walk(self.cache_directory):
            for f in files:
                if f.endswith(".lock") or f.endswith(".copy"):
                    continue
                fn = os.path.join(root, f)
                try:
                    st = os.stat(fn)
                except OSError:
                    continue
                entries.append((st.st_mtime, fn, st.st_size))
        entries.sort()
        free = usage.free
        for mtime, fn, size in entries:
            with self._lock:
                if fn in self._in_use:
                    continue
            age = now - mtime
            if age > self._always_older or (age > self._wanted_older and free < want_free):
                try:
                    os.remove(fn)
                    free += size
                except OSError:
                    pass

    def handle_cached_files_in_config(self, config: Any) -> Tuple[Any, List[str]]:
        """replace every :class:`CachedFile` in a nested structure by its local path"""
        used: List[str] = []

        def rec(x):
            if isinstance(x, CachedFile):
                p = self.get_file(x.filename)
                used.append(p)
                return p
            if isinstance(x, dict):
                return {k: rec(v) for k, v in x.items()}
            if isinstance(x, (list, tuple)):
                return type(x)(rec(v) for v in x)
            return x

        return rec(config), used


_instance: Optional[FileCache] = None


def get_instance(config=None) -> FileCache:
    """process-wide cache, options from config ``file_cache_opts``"""
    global _instance
    if _instance is None:
        opts = {}
        if config is None:
            from ..config import get_global_config

            config = get_global_config(raise_exception=False)
        if config is not None:
            opts = config.typed_value("file_cache_opts", None) or {}
        _instance = FileCache(**opts)
    return _instance


def get_instance_if_enabled() -> Optional[FileCache]:
    """the cache if ``use_file_cache`` / ``file_cache_opts`` is set in the global config"""
    from ..config import get_global_config

    config = get_global_config(raise_exception=False)
    if config is None:
        return None
    if config.has("file_cache_opts") or config.bool("use_file_cache", False):
        return get_instance(config)
    return None


def handle_cached_files_in_config(config: Any, *, file_cache: Optional[FileCache] = None):
    """module-level shortcut"""
    return (file_cache or get_instance()).handle_cached_files_in_config(config)
