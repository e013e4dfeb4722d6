"""
LRU cache decorator with direct access to the cache: peek without computing, set, pop, resize.

Parity: returnn/util/lru_cache.py (lru_cache :13; a port of the functools one with the extra accessors). This version keeps
the entries in an ``OrderedDict`` under a lock.
"""

from __future__ import annotations
from collections import OrderedDict, namedtuple
from threading import RLock
import functools

_CacheInfo = namedtuple("CacheInfo", ["hits", "misses", "maxsize", "currsize"])
_not_specified = object()
_kw_mark = object()


def _key(args, kwargs, typed):
    key = args
    if kwargs:
        key += (_kw_mark,) + tuple(sorted(kwargs.items()))
    if typed:
        key += tuple(type(a) for a in args) + tuple(type(v) for _, v in sorted(kwargs.items()))
    return key


def lru_cache(maxsize=128, typed: bool = False):
    """
    ``f.cache_info()``, ``f.cache_clear()``, ``f.cache_len()``, ``f.cache_set(*args, result, **kwargs)``,
    ``f.cache_peek(*args, update_statistics=False, fallback=None, **kwargs)``, ``f.cache_pop_oldest()``,
    ``f.cache_pop(*args, fallback=..., **kwargs)``, ``f.cache_set_maxsize(n)``, ``f.__wrapped__``.
    ``maxsize=None``: unbounded.
    """
    if callable(maxsize) and isinstance(typed, bool):
        return _wrap(maxsize, 128, typed)
    assert maxsize is None or (isinstance(maxsize, int) and maxsize >= 0)
    return lambda fn: _wrap(fn, maxsize, typed)


def _wrap(fn, maxsize, typed):
    cache: "OrderedDict" = OrderedDict()
    lock = RLock()
    stats = {"hits": 0, "misses": 0, "maxsize": maxsize}

    def _shrink():
        while stats["maxsize"] is not None and len(cache) > stats["maxsize"]:
            cache.popitem(last=False)

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        k = _key(args, kwargs, typed)
        with lock:
            if k in cache:
                cache.move_to_end(k)
                stats["hits"] += 1
                return cache[k]
            stats["misses"] += 1
        res = fn(*args, **kwargs)
        with lock:
            if stats["maxsize"] != 0:
                cache[k] = res
                cache.move_to_end(k)
                _shrink()
        return res

    def cache_peek(*args, update_statistics: bool = False, fallback=None, **kwargs):
        k = _key(args, kwargs, typed)
        with lock:
            if k in cache:
                if update_statistics:
                    stats["hits"] += 1
                    cache.move_to_end(k)
                return cache[k]
            if update_statistics:
                stats["misses"] += 1
            return fallback

    def cache_set(*args, **kwargs):
        *a, result = args
        with lock:
            if stats["maxsize"] != 0:
                k = _key(tuple(a), kwargs, typed)
                cache[k] = result
                cache.move_to_end(k)
                _shrink()

    def cache_pop(*args, fallback=_not_specified, **kwargs):
        k = _key(args, kwargs, typed)
        with lock:
            if k in cache:
                return cache.pop(k)
        if fallback is _not_specified:
            raise KeyError("not in cache: %r" % (k,))
        return fallback

    def cache_pop_oldest(*, fallback=_not_specified):
        with lock:
            if cache:
                return cache.popitem(last=False)[1]
        if fallback is _not_specified:
            raise KeyError("cache is empty")
        return fallback

    def cache_set_maxsize(new_maxsize):
        with lock:
            stats["maxsize"] = new_maxsize
            _shrink()

    def cache_clear():
        with lock:
            cache.clear()
            stats["hits"] = stats["misses"] = 0

    wrapper.cache_info = lambda: _CacheInfo(stats["hits"], stats["misses"], stats["maxsize"], len(cache))
    wrapper.cache_len = lambda: len(cache)
    wrapper.cache_clear = cache_clear
    wrapper.cache_peek = cache_peek
    wrapper.cache_set = cache_set
    wrapper.cache_pop = cache_pop
    wrapper.cache_pop_oldest = cache_pop_oldest
    wrapper.cache_set_maxsize = cache_set_maxsize
    return wrapper
