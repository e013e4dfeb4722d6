"""
Reader and writer of RASR ("Sprint") archive files: feature caches, alignment caches, bundles of archives, mixture sets and
word-boundary files; the allophone-to-label mapping that turns an alignment into class indices.

Layout of an archive, little endian throughout:

* 8 bytes ``SP_ARC1\\0``, one byte "has a table of contents".
* entries: u32 start tag ``0xAA55AA55``, u32 name length, name, then (at the entry's *position*) u32 size, u32 compressed size,
  u32 checksum, the payload (``compressed size`` bytes of a zlib/gzip stream when that is > 0, else ``size`` bytes), u32 end tag
  ``0x55AA55AA``.
* table of contents at the end: u32 count, per entry (u32 name length, name, u64 position, u32 size, u32 compressed size), a u64 zero,
  and in the last 8 bytes the u64 offset of the table. Without a table the entries are found by their start tags.
* feature payload: u32 length + ``vector-f32``, u32 frame count, per frame u32 width, width x f32, start and end time as 2 x f64.
* alignment payload: u32 length + ``flow-alignment``, u32 flags, 8 bytes ``ALIGNRLE`` (or ``AALPHRLE``), u32 size. Below 2^31 the size
  is the number of frames in a run-length code (signed byte n: n > 0 introduces n distinct u32 emissions, n < 0 one u32 emission
  that holds for -n frames, n = 0 a u32 that sets the time). Otherwise its low bits give the version (1 or 2) of the weighted code:
  packed-u32 item count, then groups (packed count*2 | time-follows bit, optional packed time, per item packed emission and a weight
  as s16/65535 (version 1) or f32 (version 2)).
* an emission index is ``allophone + state * 2**26``.

The whole file is mapped once and every entry is decoded from that buffer with ``struct.unpack_from`` / ``numpy.frombuffer``: a
feature entry costs two strided numpy views instead of one read call per value.

Parity: returnn/sprint/cache.py (``FileArchive`` :43, ``FileArchiveBundle`` :573, ``open_file_archive`` :675,
``is_sprint_cache_file`` :689, ``AllophoneLabeling`` :707, ``MixtureSet`` :807, ``WordBoundaries`` :986, ``main`` :1038).
"""

from __future__ import annotations
from typing import Dict, List, Optional, Sequence, Tuple, Union
import mmap
import os
import struct
import sys
import zlib
import numpy

_HEADER = b"SP_ARC1\0"
_START_TAG = 0xAA55AA55
_END_TAG = 0x55AA55AA
_STATE_SHIFT = 26
_MAX_STATES = 6


class FileInfo:
    """one line of the table of contents"""

    __slots__ = ("name", "pos", "size", "compressed", "index")

    def __init__(self, name: str, pos: int, size: int, compressed: int, index: int):
        self.name, self.pos, self.size, self.compressed, self.index = name, pos, size, compressed, index

    def __repr__(self):
        return "FileInfo(%r, pos=%i, size=%i, compressed=%i, index=%i)" % (self.name, self.pos, self.size, self.compressed, self.index)


class _Cursor:
    """sequential decoder over a bytes-like buffer"""

    __slots__ = ("buf", "pos")

    def __init__(self, buf, pos: int = 0):
        self.buf, self.pos = buf, pos

    def take(self, fmt: str):
        """one value of a ``struct`` format character"""
        (v,) = struct.unpack_from("<" + fmt, self.buf, self.pos)
        self.pos += struct.calcsize("<" + fmt)
        return v

    def raw(self, n: int) -> bytes:
        """the next n bytes"""
        b = bytes(self.buf[self.pos : self.pos + n])
        if len(b) != n:
            raise EOFError("archive entry ends after %i of %i bytes" % (len(b), n))
        self.pos += n
        return b

    def text(self, n: int, encoding: str = "ascii") -> str:
        """the next n bytes as a string"""
        return self.raw(n).decode(encoding)

    def packed_u32(self) -> int:
        """7 bits per byte, least significant group first, high bit = another byte follows"""
        res = shift = 0
        while True:
            b = self.buf[self.pos]
            self.pos += 1
            res |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                return res


def split_emission(emission: int, num_allophones: int) -> Tuple[int, int]:
    """:return: (allophone index, state index) of an emission index ``allophone + state * 2**26``"""
    state = 0
    while emission >= num_allophones and state < _MAX_STATES - 1:
        emission -= 1 << _STATE_SHIFT
        state += 1
    assert 0 <= emission, "emission index does not fit the allophone list"
    return emission, state


def _decode_features(cur: _Cursor) -> Tuple[List[numpy.ndarray], List[numpy.ndarray]]:
    kind = cur.text(cur.take("I"))
    assert kind == "vector-f32", "feature entry of type %r" % kind
    count = cur.take("I")
    if count == 0:
        return [], []
    width = struct.unpack_from("<I", cur.buf, cur.pos)[0]
    frame_bytes = 4 + 4 * width + 16
    block = numpy.frombuffer(cur.buf, dtype=numpy.uint8, count=count * frame_bytes, offset=cur.pos).reshape(count, frame_bytes)
    widths = block[:, :4].copy().view("<u4")[:, 0]
    if (widths == width).all():  # the usual case: every frame as wide as the first, two strided views
        feats = block[:, 4 : 4 + 4 * width].copy().view("<f4")
        times = block[:, 4 + 4 * width :].copy().view("<f8")
        cur.pos += count * frame_bytes
        return list(times), list(feats)
    times_l, feats_l = [], []
    for _ in range(count):  # frames of different widths: one by one
        w = cur.take("I")
        feats_l.append(numpy.frombuffer(cur.buf, dtype="<f4", count=w, offset=cur.pos).copy())
        cur.pos += 4 * w
        times_l.append(numpy.frombuffer(cur.buf, dtype="<f8", count=2, offset=cur.pos).copy())
        cur.pos += 16
    return times_l, feats_l


def _decode_alignment(cur: _Cursor, allophones: Sequence[str], raw: bool) -> List[Tuple[int, int, Optional[int], float]]:
    kind = cur.text(cur.take("I"))
    assert kind == "flow-alignment", "alignment entry of type %r" % kind
    cur.take("I")  # flags
    code = cur.text(8)
    if code not in ("ALIGNRLE", "AALPHRLE"):  # the second form appends its label alphabet, which is not needed here
        raise Exception("no alignment header in this entry (found %r): not an alignment cache?" % code)

    def split(e):
        if raw:
            return e, None
        assert allophones, "reading an alignment needs the allophone list (set_allophones)"
        return split_emission(e, len(allophones))

    size = cur.take("I")
    out: List[Tuple[int, int, Optional[int], float]] = []
    if size < (1 << 31):
        t = 0
        while len(out) < size:
            n = cur.take("b")
            if n > 0:
                for _ in range(n):
                    a, s = split(cur.take("I"))
                    out.append((t, a, s, 1))
                    t += 1
            elif n < 0:
                a, s = split(cur.take("I"))
                for _ in range(-n):
                    out.append((t, a, s, 1))
                    t += 1
            else:
                t = cur.take("I")
        return out
    version = size & ((1 << 31) - 1)
    assert version in (1, 2), "weighted alignment code of version %i" % version
    size = cur.packed_u32()
    t = 0
    while len(out) < size:
        n = cur.packed_u32()
        if n & 1:
            t = cur.packed_u32()
        for _ in range(n >> 1):
            a, s = split(cur.packed_u32())
            w = cur.take("h") / 65535 if version == 1 else cur.take("f")
            out.append((t, a, s, w))
        t += 1
    return out


class FileArchive:
    """
    One archive file. An existing file is opened for reading; with ``must_exists=False`` a missing file is created for writing
    (:meth:`add_feature_cache`, :meth:`add_alignment`, :meth:`add_attributes`, then :meth:`finalize` writes the table of contents).
    """

    SprintCacheHeader = _HEADER.decode("ascii")
    start_recovery_tag = _START_TAG
    end_recovery_tag = _END_TAG

    def __init__(self, filename: str, must_exists: bool = True, encoding: str = "ascii"):
        self.filename = filename
        self.encoding = encoding
        self.ft: Dict[str, FileInfo] = {}
        self.allophones: List[str] = []
        self._buf = None
        self._out = None
        if os.path.exists(filename):
            with open(filename, "rb") as f:
                self._buf = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(filename) else b""
            assert bytes(self._buf[:8]) == _HEADER, "%s: not a Sprint archive" % filename
            if self._buf[8]:
                self._read_table()
            else:
                self._scan()
        else:
            assert not must_exists, "File does not exist: %r" % filename
            self._out = open(filename, "wb")
            self._out.write(_HEADER + b"\x01")
        self._index_short_names()

    def _index_short_names(self):
        self._short_seg_names = {os.path.basename(n): n for n in self.ft}
        if len(self._short_seg_names) < len(self.ft):  # base names collide: no lookup by base name
            self._short_seg_names = {}

    def __repr__(self):
        return "<%s %r %i entries>" % (type(self).__name__, self.filename, len(self.ft))

    def _read_table(self):
        (table_pos,) = struct.unpack_from("<Q", self._buf, len(self._buf) - 8)
        cur = _Cursor(self._buf, table_pos)
        for i in range(cur.take("I")):
            name = cur.text(cur.take("I"), self.encoding)
            pos, size, comp = cur.take("Q"), cur.take("I"), cur.take("I")
            self.ft[name] = FileInfo(name, pos, size, comp, i)

    def _scan(self):
        """no table of contents: walk the start tags"""
        tag = struct.pack("<I", _START_TAG)
        at = self._buf.find(tag, 0) if hasattr(self._buf, "find") else -1
        while at >= 0:
            cur = _Cursor(self._buf, at + 4)
            try:
                name = cur.text(cur.take("I"), self.encoding)
                pos = cur.pos
                size, comp = cur.take("I"), cur.take("I")
                cur.take("I")  # checksum
            except (struct.error, EOFError, UnicodeDecodeError):
                at = self._buf.find(tag, at + 1)
                continue
            self.ft[name] = FileInfo(name, pos, size, comp, len(self.ft))
            at = self._buf.find(tag, cur.pos + (comp or size))

    def file_list(self):
        """:return: names of all entries (attribute entries ``*.attribs`` included)"""
        return self.ft.keys()

    def has_entry(self, filename: str) -> bool:
        """:return: whether :meth:`read` knows this name"""
        return filename in self.ft

    def _payload(self, filename: str) -> Tuple[Optional[_Cursor], FileInfo]:
        if filename not in self.ft and filename in self._short_seg_names:
            filename = self._short_seg_names[filename]
        info = self.ft[filename]
        cur = _Cursor(self._buf, info.pos)
        size, comp = cur.take("I"), cur.take("I")
        cur.take("I")  # checksum
        if size == 0:
            return None, info
        if comp > 0:
            return _Cursor(zlib.decompress(cur.raw(comp), 15 + 32)), info  # zlib or gzip wrapper, detected from the stream
        return cur, info

    def read(self, filename: str, typ: str):
        """
        :param filename: entry name (or its base name, where base names are unique)
        :param typ: "str", "feat", "align" or "align_raw"
        :return: "str": the text. "feat": (times, features), one [start, end] float64 pair and one float32 vector per frame.
            "align": list of (time, allophone index, state index, weight). "align_raw": the same with the undivided emission
            index in place of the allophone and None for the state. None for an empty entry.
        """
        assert self._buf is not None, "%r is open for writing" % self
        cur, info = self._payload(filename)
        if cur is None:
            return None
        if typ == "str":
            return cur.text(info.size, self.encoding)
        if typ == "feat":
            return _decode_features(cur)
        if typ in ("align", "align_raw"):
            return _decode_alignment(cur, self.allophones, raw=typ == "align_raw")
        raise ValueError("%r: unknown typ %r" % (self, typ))

    def get_state(self, mix: int) -> Tuple[int, int]:
        """:return: (allophone index, state index) for an emission index"""
        assert self.allophones
        return split_emission(mix, len(self.allophones))

    def set_allophones(self, f: str):
        """:param f: allophone file, one per line, ``#`` lines are comments"""
        self.allophones[:] = [ln.strip() for ln in open(f) if not ln.strip().startswith("#")]

    def get_allophones_list(self) -> List[str]:
        """:return: the allophones set before"""
        return self.allophones

    # -- writing --

    def _add_entry(self, name: str, payload: bytes, compress: bool = False):
        assert self._out is not None, "%r is open for reading" % self
        raw_name = name.encode(self.encoding)
        self._out.write(struct.pack("<II", _START_TAG, len(raw_name)) + raw_name)
        pos = self._out.tell()
        stored = zlib.compress(payload) if compress else payload
        self._out.write(struct.pack("<III", len(payload), len(stored) if compress else 0, 0))
        self._out.write(stored)
        self._out.write(struct.pack("<I", _END_TAG))
        self.ft[name] = FileInfo(name, pos, len(payload), len(stored) if compress else 0, len(self.ft))

    def add_feature_cache(self, filename: str, features, times, compress: bool = False):
        """
        :param filename: entry name
        :param features: [T, D] array or list of vectors
        :param times: per frame (start, end)
        """
        feats = numpy.asarray(features, dtype="<f4").reshape(len(features), -1)
        tms = numpy.asarray(times, dtype="<f8").reshape(len(times), 2) if len(times) else numpy.zeros((0, 2), "<f8")
        assert len(feats) == len(tms)
        n, dim = feats.shape
        frames = numpy.zeros((n, 4 + 4 * dim + 16), dtype=numpy.uint8)
        frames[:, :4] = numpy.frombuffer(struct.pack("<I", dim), dtype=numpy.uint8)
        frames[:, 4 : 4 + 4 * dim] = feats.view(numpy.uint8).reshape(n, 4 * dim)
        frames[:, 4 + 4 * dim :] = tms.view(numpy.uint8).reshape(n, 16)
        self._add_entry(filename, struct.pack("<I", 10) + b"vector-f32" + struct.pack("<I", n) + frames.tobytes(), compress=compress)
        self.add_attributes(filename, dim if n else 0, float(tms[-1, 1]) if n else 1.0)

    def add_alignment(self, filename: str, emissions: Sequence[int], weights: Optional[Sequence[float]] = None, compress: bool = False):
        """
        :param filename: entry name
        :param emissions: per frame ``allophone + state * 2**26``
        :param weights: per frame; given, the entry uses the weighted code (version 2), else the run-length code
        """
        head = struct.pack("<I", 14) + b"flow-alignment" + struct.pack("<I", 0) + b"ALIGNRLE"
        body = bytearray()
        if weights is None:
            body += struct.pack("<I", len(emissions))
            i = 0
            while i < len(emissions):
                j = i
                while j + 1 < len(emissions) and emissions[j + 1] == emissions[i] and j + 1 - i < 127:
                    j += 1
                if j > i:  # a run
                    body += struct.pack("<bI", -(j - i + 1), emissions[i])
                    i = j + 1
                    continue
                k = i  # distinct values up to the next run
                while k + 1 < len(emissions) and k + 1 - i < 127 and not (k + 2 < len(emissions) and emissions[k + 1] == emissions[k + 2]):
                    k += 1
                body += struct.pack("<b", k - i + 1) + b"".join(struct.pack("<I", e) for e in emissions[i : k + 1])
                i = k + 1
        else:
            assert len(weights) == len(emissions)

            def packed(v):
                out = bytearray()
                while True:
                    if v < 0x80:
                        out.append(v)
                        return bytes(out)
                    out.append((v & 0x7F) | 0x80)
                    v >>= 7

            body += struct.pack("<I", (1 << 31) | 2) + packed(len(emissions))
            for e, w in zip(emissions, weights):
                body += packed(2) + packed(int(e)) + struct.pack("<f", w)
        self._add_entry(filename, head + bytes(body), compress=compress)

    def add_attributes(self, filename: str, dim: int, duration: float):
        """the ``<name>.attribs`` entry RASR keeps beside a feature entry"""
        text = ('<flow-attributes><flow-attribute name="datatype" value="vector-f32"/><flow-attribute name="sample-size" value="%d"/>'
                '<flow-attribute name="total-duration" value="%.5f"/></flow-attributes>') % (dim, duration)
        self._add_entry(filename + ".attribs", text.encode("ascii"))

    def finalize(self):
        """write the table of contents and close the file (written archives only)"""
        if self._out is None:
            return
        pos = self._out.tell()
        self._out.write(struct.pack("<I", len(self.ft)))
        for fi in self.ft.values():
            raw_name = fi.name.encode(self.encoding)
            self._out.write(struct.pack("<I", len(raw_name)) + raw_name + struct.pack("<QII", fi.pos, fi.size, fi.compressed))
        self._out.write(struct.pack("<QQ", 0, pos))
        self._out.close()
        self._out = None
        self._index_short_names()


class FileArchiveBundle:
    """several archives behind one name space; a ``.bundle`` file lists one archive per line (relative to the bundle's folder)"""

    def __init__(self, filename: Optional[str] = None, encoding: str = "ascii"):
        self.archives: Dict[str, FileArchive] = {}
        self.files: Dict[str, FileArchive] = {}
        self._short_seg_names: Dict[str, str] = {}
        if filename is not None:
            self.add_bundle(filename, encoding=encoding)

    def add_bundle(self, filename: str, encoding: str = "ascii"):
        """:param filename: bundle file"""
        base = os.path.dirname(filename) or "."
        for line in open(filename).read().splitlines():
            if line.strip():
                self.add_archive(line if line.startswith("/") else base + "/" + line, encoding=encoding)

    def add_archive(self, filename: str, encoding: str = "ascii"):
        """:param filename: single archive"""
        if filename in self.archives:
            return
        arc = self.archives[filename] = FileArchive(filename, must_exists=True, encoding=encoding)
        for name in arc.ft:
            self.files[name] = arc
        self._short_seg_names.update(arc._short_seg_names)

    def add_bundle_or_archive(self, filename: str, encoding: str = "ascii"):
        """by the file name's ending"""
        (self.add_bundle if filename.endswith(".bundle") else self.add_archive)(filename, encoding=encoding)

    @property
    def ft(self) -> Dict[str, FileInfo]:
        """the tables of contents of all archives as one"""
        return {name: arc.ft[name] for name, arc in self.files.items()}

    def file_list(self):
        """:return: all entry names"""
        return self.files.keys()

    def has_entry(self, filename: str) -> bool:
        """:return: whether an archive holds it"""
        return filename in self.files

    def read(self, filename: str, typ: str):
        """as :meth:`FileArchive.read`"""
        if filename not in self.files and filename in self._short_seg_names:
            filename = self._short_seg_names[filename]
        return self.files[filename].read(filename, typ)

    def set_allophones(self, filename: str):
        """for every archive"""
        for arc in self.archives.values():
            arc.set_allophones(filename)

    def get_allophones_list(self) -> List[str]:
        """of the first archive"""
        return next(iter(self.archives.values())).get_allophones_list()


def open_file_archive(archive_filename: str, must_exists: bool = True, encoding: str = "ascii") -> Union[FileArchive, FileArchiveBundle]:
    """a bundle for ``*.bundle``, else a single archive"""
    if archive_filename.endswith(".bundle"):
        assert must_exists
        return FileArchiveBundle(archive_filename, encoding=encoding)
    return FileArchive(archive_filename, must_exists=must_exists, encoding=encoding)


def is_sprint_cache_file(filename: str) -> bool:
    """:return: whether :func:`open_file_archive` can open this (existing) file"""
    assert os.path.exists(filename)
    if not os.path.isfile(filename):
        return False
    if filename.endswith(".bundle"):
        return True
    with open(filename, "rb") as f:
        return f.read(len(_HEADER)) == _HEADER


class AllophoneLabeling:
    """
    Maps (allophone, HMM state) to a class label: through a state-tying file (``<allophone>.<state> <label>`` per line), or, without
    one, to the index of the allophone's central phoneme in the phoneme list.
    """

    def __init__(self, silence_phone: str, allophone_file: str, phoneme_file: Optional[str] = None, state_tying_file: Optional[str] = None,
                 verbose_out=None):
        assert phoneme_file or state_tying_file
        self.allophone_file = allophone_file
        self.allophones = [ln for ln in open(allophone_file).read().splitlines() if ln and not ln.startswith("#")]
        self.allophones_idx = {a: i for i, a in enumerate(self.allophones)}
        sil = silence_phone + "{#+#}@i@f"
        self.sil_allo_state_id = self.allophones_idx[sil]
        self.phonemes = self.phoneme_idxs = self.state_tying = self.state_tying_by_allo_state_idx = None
        self.sil_label_idx = self.num_labels = self.num_allo_states = None
        if verbose_out:
            print("AllophoneLabeling: Num allophones: %i" % len(self.allophones), file=verbose_out)
        if phoneme_file:
            self.phonemes = open(phoneme_file).read().splitlines()
            self.phoneme_idxs = {p: i for i, p in enumerate(self.phonemes)}
            if not state_tying_file:
                self.sil_label_idx = self.phoneme_idxs[silence_phone]
                self.num_labels = len(self.phonemes)
        if state_tying_file:
            self.state_tying = {}
            for ln in open(state_tying_file).read().splitlines():
                if ln.strip():
                    key, label = ln.split()
                    self.state_tying[key] = int(label)
            self.sil_label_idx = self.state_tying[sil + ".0"]
            self.num_allo_states = 1 + max(int(k.rsplit(".", 1)[1]) for k in self.state_tying)
            self.state_tying_by_allo_state_idx = {}
            for a, name in enumerate(self.allophones):
                for s in range(self.num_allo_states):
                    label = self.state_tying.get("%s.%i" % (name, s))
                    if label is not None:
                        self.state_tying_by_allo_state_idx[a + (s << _STATE_SHIFT)] = label
            self.num_labels = 1 + max(self.state_tying.values())
        if verbose_out:
            print("AllophoneLabeling: %i labels." % self.num_labels, file=verbose_out)
        assert self.num_labels is not None

    def get_label_idx_by_allo_state_idx(self, allo_state_idx: int) -> int:
        """:param allo_state_idx: ``allophone + state * 2**26``"""
        if self.state_tying_by_allo_state_idx:
            return self.state_tying_by_allo_state_idx[allo_state_idx]
        return self.get_label_idx(*split_emission(allo_state_idx, len(self.allophones)))

    def get_label_idx(self, allo_idx: int, state_idx: int) -> int:
        """:return: class label"""
        if self.state_tying_by_allo_state_idx:
            key = allo_idx + (state_idx << _STATE_SHIFT)
            if key not in self.state_tying_by_allo_state_idx:
                raise KeyError("allophone %i (%r), state %i: not in the state tying" % (allo_idx, self.allophones[allo_idx], state_idx))
            return self.state_tying_by_allo_state_idx[key]
        name = self.allophones[allo_idx]
        return self.phoneme_idxs[name[: name.index("{")]]


class MixtureSet:
    """
    Gaussian mixture set file: ``MIXSET\\0`` + one byte, u32 version, u32 dim, then four counted tables: means and covariances (each
    u32 dim, dim x f64, f64 weight), densities (u32 mean index, u32 covariance index), mixtures (u32 count, count x (u32 density, f64
    weight)).
    """

    header = "MIXSET\0"

    def __init__(self, filename: Optional[str] = None):
        self.version = 0
        self.dim = 0
        self.means = numpy.zeros((0, 0))
        self.mean_weights = numpy.zeros((0,))
        self.covs = numpy.zeros((0, 0))
        self.cov_weights = numpy.zeros((0,))
        self.densities = numpy.zeros((0, 2), dtype=numpy.int32)
        self.mixtures: List[Tuple[List[int], List[float]]] = []
        if filename is not None:
            self._load(filename)

    def _load(self, filename: str):
        cur = _Cursor(open(filename, "rb").read())
        assert cur.text(8)[:7] == self.header, "%s: not a mixture set" % filename
        self.version, self.dim = cur.take("I"), cur.take("I")

        def table():
            n = cur.take("I")
            rec = numpy.dtype([("dim", "<u4"), ("v", "<f8", (self.dim,)), ("w", "<f8")])
            arr = numpy.frombuffer(cur.buf, dtype=rec, count=n, offset=cur.pos)
            cur.pos += n * rec.itemsize
            assert (arr["dim"] == self.dim).all()
            return arr["v"].astype(numpy.float64), arr["w"].astype(numpy.float64)

        self.means, self.mean_weights = table()
        self.covs, self.cov_weights = table()
        n = cur.take("I")
        self.densities = numpy.frombuffer(cur.buf, dtype="<u4", count=2 * n, offset=cur.pos).reshape(n, 2).astype(numpy.int32)
        cur.pos += 8 * n
        self.mixtures = []
        for _ in range(cur.take("I")):
            k = cur.take("I")
            rec = numpy.frombuffer(cur.buf, dtype=numpy.dtype([("d", "<u4"), ("w", "<f8")]), count=k, offset=cur.pos)
            cur.pos += 12 * k
            self.mixtures.append(([int(x) for x in rec["d"]], [float(x) for x in rec["w"]]))

    num_means = property(lambda self: len(self.means))
    num_covs = property(lambda self: len(self.covs))
    num_densities = property(lambda self: len(self.densities))
    num_mixtures = property(lambda self: len(self.mixtures))

    def write(self, filename: str):
        """in the layout :meth:`__init__` reads"""
        with open(filename, "wb") as f:
            f.write(self.header.encode("ascii") + b"t" + struct.pack("<II", self.version, self.dim))
            for vecs, weights in ((self.means, self.mean_weights), (self.covs, self.cov_weights)):
                f.write(struct.pack("<I", len(vecs)))
                for v, w in zip(vecs, weights):
                    f.write(struct.pack("<I", self.dim) + numpy.asarray(v, "<f8").tobytes() + struct.pack("<d", w))
            f.write(struct.pack("<I", len(self.densities)) + numpy.asarray(self.densities, "<u4").tobytes())
            f.write(struct.pack("<I", len(self.mixtures)))
            for idx, weights in self.mixtures:
                f.write(struct.pack("<I", len(idx)) + b"".join(struct.pack("<Id", i, w) for i, w in zip(idx, weights)))

    def get_mean_by_idx(self, idx: int) -> numpy.ndarray:
        """mean of the first density of mixture idx"""
        return numpy.float32(self.means[self.densities[self.mixtures[idx][0][0], 0]])

    def get_cov_by_idx(self, idx: int) -> numpy.ndarray:
        """covariance (diagonal) of the first density of mixture idx"""
        return numpy.float32(self.covs[self.densities[self.mixtures[idx][0][0], 1]])

    def get_number_mixtures(self) -> int:
        """:return: number of mixtures"""
        return self.num_mixtures


class WordBoundaries:
    """lattice word-boundary file: ``LATWRDBN``, u32 version, u32 count, per boundary u32 time, u16 final, u16 initial"""

    header = "LATWRDBN"

    def __init__(self, filename: str, verbose_out=None):
        cur = _Cursor(open(filename, "rb").read())
        assert cur.text(8) == self.header, "%s: not a word-boundary file" % filename
        self.version, self.size = cur.take("I"), cur.take("I")
        rec = numpy.frombuffer(cur.buf, dtype=numpy.dtype([("t", "<u4"), ("f", "<u2"), ("i", "<u2")]), count=self.size, offset=cur.pos)
        self.boundaries = [(int(r["t"]), int(r["i"]), int(r["f"])) for r in rec]  # (time, initial, final)
        if verbose_out:
            print("version=%d size=%d" % (self.version, self.size), file=verbose_out)
            for b in self.boundaries:
                print(b, file=verbose_out)


def main(argv: Optional[Sequence[str]] = None):
    """``python -m returnn_b200.sprint.cache <archive> [<entry>] [--mode list|show] [--type feat|align] [--allophone-file F]``"""
    from argparse import ArgumentParser

    ap = ArgumentParser(description="list or show the entries of a Sprint archive")
    ap.add_argument("archive")
    ap.add_argument("file", nargs="?")
    ap.add_argument("--mode", default="list", help="list, show")
    ap.add_argument("--type", default="feat", help="feat, align, ascii")
    ap.add_argument("--allophone-file")
    args = ap.parse_args(argv)
    arc = open_file_archive(args.archive, must_exists=True)
    if args.mode == "list":
        print("\n".join(sorted(arc.file_list())))
        return
    assert args.mode == "show", "invalid --mode %r" % args.mode
    assert args.file, "--mode show needs the entry name"
    if args.type == "align":
        if args.allophone_file:
            arc.set_allophones(args.allophone_file)
        for t, index, state, weight in arc.read(args.file, "align"):
            items = ["time=%i" % t, "allophone=%s" % arc.get_allophones_list()[index], "index=%i" % index, "state=%s" % state]
            if weight != 1:
                items.append("weight=%s" % weight)
            print("\t".join(items))
    elif args.type == "feat":
        times, feats = arc.read(args.file, "feat")
        for tm, row in zip(times, feats):
            print("%s--------%s" % (tm, " ".join("%.6f " % x for x in row)))
    elif args.type == "ascii":
        print(arc.read(args.file, "str"))
    else:
        raise NotImplementedError("invalid --type %r" % args.type)


if __name__ == "__main__":
    main(sys.argv[1:])
