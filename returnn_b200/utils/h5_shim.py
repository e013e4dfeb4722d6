"""
A small stand-in for the part of the ``h5py`` API that the dataset code uses, for machines without HDF5.

``get_h5py()`` returns the real ``h5py`` when it can be imported and this module otherwise. The stand-in keeps the same object
model (``File`` -> groups -> datasets with ``shape`` / ``dtype`` / slicing / ``resize`` / ``attrs``), so the dataset readers and
writers run the same code in both cases; only the container differs: a file written by the stand-in is a numpy ``.npz`` archive
(one array per dataset path, attributes as JSON), not an HDF5 file. Opening a real HDF5 file (recognised by its signature)
without ``h5py`` raises an error that says so.
"""

from __future__ import annotations
from typing import Any, Dict, Iterator, List, Optional, Tuple, Union
import io
import json
import os
import numpy

_HDF5_SIGNATURE = b"\x89HDF\r\n\x1a\n"


def get_h5py():
    """the ``h5py`` module, or this module as its stand-in"""
    try:
        import h5py  # noqa

        return h5py
    except ImportError:
        import sys

        return sys.modules[__name__]


def have_real_h5py() -> bool:
    """whether files are real HDF5"""
    try:
        import h5py  # noqa: F401

        return True
    except ImportError:
        return False


def special_dtype(vlen=None, **_kwargs):
    """variable-length string type (``h5py.special_dtype(vlen=str)``): numpy object arrays of str here"""
    return numpy.dtype(object)


def string_dtype(encoding: str = "utf-8", length=None):
    """``h5py.string_dtype``"""
    return numpy.dtype(object)


class AttributeManager(dict):
    """``obj.attrs``"""

    def create(self, name, data, shape=None, dtype=None):
        """h5py-style explicit creation"""
        self[name] = numpy.asarray(data, dtype=dtype)

    def modify(self, name, value):
        """overwrite"""
        self[name] = value


class Dataset:
    """an array with h5py's dataset surface"""

    def __init__(self, name: str, data: numpy.ndarray, maxshape=None):
        self.name = name
        self._data = data
        self.maxshape = maxshape
        self.attrs = AttributeManager()

    @property
    def shape(self) -> Tuple[int, ...]:
        """current shape"""
        return self._data.shape

    @property
    def dtype(self):
        """numpy dtype"""
        return self._data.dtype

    @property
    def ndim(self) -> int:
        """number of axes"""
        return self._data.ndim

    @property
    def size(self) -> int:
        """number of elements"""
        return self._data.size

    def __len__(self):
        return len(self._data)

    def __getitem__(self, key):
        out = self._data[key]
        if isinstance(out, numpy.ndarray):
            return out.copy()
        return out

    def __setitem__(self, key, value):
        self._data[key] = value

    def __iter__(self):
        return iter(self._data)

    def __array__(self, dtype=None, copy=None):
        return numpy.asarray(self._data, dtype=dtype)

    def resize(self, size, axis: Optional[int] = None):
        """grow or shrink (new entries are zero / empty)"""
        if axis is not None:
            new_shape = list(self._data.shape)
            new_shape[axis] = int(size)
        else:
            new_shape = list(size) if isinstance(size, (tuple, list)) else [int(size)] + list(self._data.shape[1:])
        new = numpy.zeros(new_shape, dtype=self._data.dtype)
        if self._data.dtype == object:
            new[...] = ""
        common = tuple(slice(0, min(a, b)) for a, b in zip(self._data.shape, new_shape))
        new[common] = self._data[common]
        self._data = new

    def asstr(self):
        """h5py's view of a string dataset as str"""
        return self

    def read_direct(self, dest, source_sel=None, dest_sel=None):
        """copy into an existing array"""
        dest[dest_sel if dest_sel is not None else Ellipsis] = self._data[source_sel if source_sel is not None else Ellipsis]


class Group:
    """a node with children"""

    def __init__(self, name: str = "/"):
        self.name = name
        self._children: Dict[str, Union["Group", Dataset]] = {}
        self.attrs = AttributeManager()

    # -- lookup
    def _split(self, path: str) -> List[str]:
        return [p for p in path.split("/") if p]

    def __contains__(self, path: str) -> bool:
        node: Any = self
        for part in self._split(path):
            if not isinstance(node, Group) or part not in node._children:
                return False
            node = node._children[part]
        return True

    def __getitem__(self, path: str):
        node: Any = self
        for part in self._split(path):
            if not isinstance(node, Group) or part not in node._children:
                raise KeyError("unable to open object %r in %r" % (path, self.name))
            node = node._children[part]
        return node

    def get(self, path: str, default=None):
        """like dict.get"""
        return self[path] if path in self else default

    def __iter__(self) -> Iterator[str]:
        return iter(sorted(self._children))

    def __len__(self):
        return len(self._children)

    def keys(self):
        """child names"""
        return sorted(self._children)

    def values(self):
        """children"""
        return [self._children[k] for k in self.keys()]

    def items(self):
        """(name, child)"""
        return [(k, self._children[k]) for k in self.keys()]

    def __delitem__(self, path: str):
        parts = self._split(path)
        parent = self["/".join(parts[:-1])] if len(parts) > 1 else self
        del parent._children[parts[-1]]

    # -- creation
    def _parent_of(self, path: str, create: bool) -> Tuple["Group", str]:
        parts = self._split(path)
        node = self
        for part in parts[:-1]:
            if part not in node._children:
                if not create:
                    raise KeyError(path)
                node._children[part] = Group((node.name.rstrip("/") + "/" + part))
            node = node._children[part]  # type: ignore
            assert isinstance(node, Group)
        return node, parts[-1]

    def create_group(self, path: str) -> "Group":
        """new (nested) group"""
        parent, leaf = self._parent_of(path, create=True)
        if leaf in parent._children:
            raise ValueError("unable to create group %r (name already exists)" % path)
        grp = Group(parent.name.rstrip("/") + "/" + leaf)
        parent._children[leaf] = grp
        return grp

    def require_group(self, path: str) -> "Group":
        """existing or new group"""
        return self[path] if path in self else self.create_group(path)

    def create_dataset(self, name: str, shape=None, dtype=None, data=None, maxshape=None, **_storage_opts) -> Dataset:
        """new dataset from ``data`` or zero-filled of ``shape`` (chunking / compression options are accepted and ignored)"""
        path = name
        parent, leaf = self._parent_of(path, create=True)
        if leaf in parent._children:
            raise ValueError("unable to create dataset %r (name already exists)" % path)
        if data is not None:
            if dtype is not None and numpy.dtype(dtype) == object:
                arr = numpy.empty(numpy.shape(data), dtype=object)
                arr[...] = [x.decode("utf8") if isinstance(x, bytes) else x for x in numpy.asarray(data, dtype=object).reshape(-1)] if numpy.ndim(data) else data
                arr = arr.reshape(numpy.shape(data))
            else:
                arr = numpy.array(data, dtype=dtype)
            if shape is not None and tuple(numpy.atleast_1d(shape)) != arr.shape:
                arr = arr.reshape(shape)
        else:
            assert shape is not None, "create_dataset: need data or shape"
            shape = (shape,) if isinstance(shape, int) else tuple(shape)
            arr = numpy.zeros(shape, dtype=dtype or "float32")
            if arr.dtype == object:
                arr[...] = ""
        ds = Dataset(parent.name.rstrip("/") + "/" + leaf, arr, maxshape=maxshape)
        parent._children[leaf] = ds
        return ds

    def __setitem__(self, path: str, value):
        self.create_dataset(path, data=value)

    def visititems(self, func):
        """depth-first over all descendants: ``func(relative_path, obj)``"""

        def walk(node: "Group", prefix: str):
            for k in node.keys():
                child = node._children[k]
                rel = prefix + k
                res = func(rel, child)
                if res is not None:
                    return res
                if isinstance(child, Group):
                    res = walk(child, rel + "/")
                    if res is not None:
                        return res
            return None

        return walk(self, "")


class File(Group):
    """``File(path, mode)`` with modes r, r+, a, w, w- / x"""

    def __init__(self, filename: str, mode: str = "r", **_kwargs):
        super().__init__("/")
        self.filename = str(filename)
        self.mode = mode
        self._closed = False
        exists = os.path.exists(self.filename)
        if mode in ("r", "r+") and not exists:
            raise FileNotFoundError("unable to open file %r (no such file)" % self.filename)
        if mode in ("w-", "x") and exists:
            raise FileExistsError("unable to create file %r (file exists)" % self.filename)
        if exists and mode in ("r", "r+", "a"):
            self._load()

    def _load(self):
        with open(self.filename, "rb") as f:
            head = f.read(8)
        if head == _HDF5_SIGNATURE:
            raise ImportError("%r is a real HDF5 file; reading it needs the h5py package, which is not installed here" % self.filename)
        with numpy.load(self.filename, allow_pickle=True) as z:
            meta = json.loads(str(z["__meta__"])) if "__meta__" in z.files else {"groups": [], "attrs": {}}
            for g in meta.get("groups", []):
                self.require_group(g)
            for key in z.files:
                if key == "__meta__":
                    continue
                path = key.replace("|", "/")
                ds = self.create_dataset(path, data=z[key])
                ds._data = z[key]
            for path, attrs in meta.get("attrs", {}).items():
                node = self if path in ("", "/") else self[path]
                for k, v in attrs.items():
                    node.attrs[k] = numpy.array(v["value"], dtype=v["dtype"]) if v.get("array") else v["value"]

    def flush(self):
        """write the tree to disk (modes other than r)"""
        if self.mode == "r" or self._closed:
            return
        arrays: Dict[str, numpy.ndarray] = {}
        groups: List[str] = []
        attrs: Dict[str, Dict[str, Any]] = {}

        def enc_attrs(path: str, node):
            if node.attrs:
                out = {}
                for k, v in node.attrs.items():
                    if isinstance(v, numpy.ndarray):
                        out[k] = {"array": True, "dtype": str(v.dtype), "value": v.tolist()}
                    elif isinstance(v, (numpy.generic,)):
                        out[k] = {"value": v.item()}
                    elif isinstance(v, bytes):
                        out[k] = {"value": v.decode("utf8")}
                    else:
                        out[k] = {"value": v}
                attrs[path] = out

        enc_attrs("/", self)

        def visit(rel: str, obj):
            if isinstance(obj, Group):
                groups.append(rel)
            else:
                arrays[rel.replace("/", "|")] = obj._data
            enc_attrs(rel, obj)

        self.visititems(visit)
        meta = json.dumps({"groups": groups, "attrs": attrs})
        buf = io.BytesIO()
        numpy.savez(buf, __meta__=numpy.array(meta), **arrays)
        tmp = self.filename + ".tmp.%i" % os.getpid()
        with open(tmp, "wb") as f:
            f.write(buf.getvalue())
        os.replace(tmp, self.filename)

    def close(self):
        """flush and close"""
        if not self._closed:
            self.flush()
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def is_hdf5(filename: str) -> bool:
    """whether the file carries the HDF5 signature"""
    try:
        with open(filename, "rb") as f:
            return f.read(8) == _HDF5_SIGNATURE
    except OSError:
        return False
