"""
Minimal pure-Python stand-in for the ``dm-tree`` package (``import tree``), which the reference imports but which is
not installed in this image. Only used to run the reference arm of ``bench.py``; it is put on ``sys.path`` after the
reference itself. Semantics follow dm-tree: dicts are traversed in sorted key order, lists / tuples / namedtuples in
order, everything else (including None) is a leaf.
"""

from __future__ import annotations
import collections.abc

__all__ = ["is_nested", "flatten", "flatten_with_path", "unflatten_as", "map_structure", "map_structure_with_path",
           "assert_same_structure", "map_structure_up_to", "traverse"]


def _is_namedtuple(x) -> bool:
    return isinstance(x, tuple) and hasattr(x, "_fields")


def is_nested(x) -> bool:
    """whether x is a container dm-tree would traverse"""
    return isinstance(x, (list, tuple, collections.abc.Mapping)) and not isinstance(x, (str, bytes))


def _sorted_keys(d):
    try:
        return sorted(d.keys())
    except TypeError:
        return list(d.keys())


def _children(x):
    if isinstance(x, collections.abc.Mapping):
        return [(k, x[k]) for k in _sorted_keys(x)]
    if _is_namedtuple(x):
        return list(zip(x._fields, x))
    return list(enumerate(x))


def _rebuild(x, values):
    if isinstance(x, collections.abc.Mapping):
        keys = _sorted_keys(x)
        mapping = dict(zip(keys, values))
        try:
            res = type(x)()
            for k in x.keys():
                res[k] = mapping[k]
            return res
        except Exception:
            return {k: mapping[k] for k in x.keys()}
    if _is_namedtuple(x):
        return type(x)(*values)
    return type(x)(values)


def flatten(structure):
    """leaves in traversal order"""
    out = []

    def rec(x):
        if is_nested(x):
            for _, v in _children(x):
                rec(v)
        else:
            out.append(x)

    rec(structure)
    return out


def flatten_with_path(structure):
    """[(path tuple, leaf)]"""
    out = []

    def rec(x, path):
        if is_nested(x):
            for k, v in _children(x):
                rec(v, path + (k,))
        else:
            out.append((path, x))

    rec(structure, ())
    return out


def unflatten_as(structure, flat_sequence):
    """inverse of flatten"""
    it = iter(flat_sequence)

    def rec(x):
        if is_nested(x):
            return _rebuild(x, [rec(v) for _, v in _children(x)])
        return next(it)

    return rec(structure)


def assert_same_structure(a, b, check_types: bool = True):
    """raise ValueError / TypeError when the nestings differ"""
    if is_nested(a) != is_nested(b):
        raise ValueError("The two structures don't have the same nested structure: %r vs %r" % (a, b))
    if not is_nested(a):
        return
    if check_types and type(a) is not type(b):
        if not (isinstance(a, collections.abc.Mapping) and isinstance(b, collections.abc.Mapping)):
            raise TypeError("The two structures don't have the same sequence type: %s vs %s" % (type(a), type(b)))
    ca, cb = _children(a), _children(b)
    if len(ca) != len(cb) or [k for k, _ in ca] != [k for k, _ in cb]:
        raise ValueError("The two structures don't have the same nested structure: %r vs %r" % (a, b))
    for (_, va), (_, vb) in zip(ca, cb):
        assert_same_structure(va, vb, check_types=check_types)


def map_structure(func, *structures, check_types: bool = True):
    """apply func leaf-wise over parallel structures"""
    if not callable(func):
        raise TypeError("func must be callable, got: %r" % (func,))
    if not structures:
        raise ValueError("Must provide at least one structure")
    for other in structures[1:]:
        assert_same_structure(structures[0], other, check_types=check_types)
    flats = [flatten(s) for s in structures]
    return unflatten_as(structures[0], [func(*xs) for xs in zip(*flats)])


def map_structure_with_path(func, *structures, check_types: bool = True):
    """like map_structure; func gets the path first"""
    for other in structures[1:]:
        assert_same_structure(structures[0], other, check_types=check_types)
    paths = [p for p, _ in flatten_with_path(structures[0])]
    flats = [flatten(s) for s in structures]
    return unflatten_as(structures[0], [func(p, *xs) for p, xs in zip(paths, zip(*flats))])


def map_structure_up_to(shallow_structure, func, *structures, check_types: bool = True):
    """map only down to the depth of shallow_structure"""

    def rec(shallow, *subs):
        if is_nested(shallow):
            kids = _children(shallow)
            sub_kids = [dict(_children(s)) for s in subs]
            return _rebuild(shallow, [rec(v, *[sk[k] for sk in sub_kids]) for k, v in kids])
        return func(*subs)

    return rec(shallow_structure, *structures)


def traverse(fn, structure, top_down: bool = True):
    """visit every sub-structure; fn may return a replacement"""

    def rec(x):
        if top_down:
            r = fn(x)
            if r is not None:
                return r
        if is_nested(x):
            x = _rebuild(x, [rec(v) for _, v in _children(x)])
        if not top_down:
            r = fn(x)
            if r is not None:
                return r
        return x

    return rec(structure)
