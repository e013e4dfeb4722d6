"""
:class:`OggZipDataset`: a zip file (or directory) with audio files and a ``<name>.txt`` listing
``[{"file": ..., "text": ..., "duration": ..., "seq_name": ...}, ...]``; features are extracted on the fly
(reference: returnn/datasets/audio.py:18). Keys: ``data`` (features, unless ``audio=None``), ``classes`` (targets from
the vocabulary, unless ``targets=None``), ``orth`` (utf8 bytes), ``raw`` (text as numpy string).

Decoding: ``.wav`` through the standard library; ``.ogg`` / ``.flac`` need the ``soundfile`` package (optional).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Union
import ast
import io
import os
import wave
import zipfile
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from .util.vocabulary import Vocabulary
from .util.feature_extraction import ExtractAudioFeatures


def read_audio(raw: bytes, name: str):
    """:return: (float32 samples [n] or [n, ch], sample_rate)"""
    if name.lower().endswith(".wav"):
        with wave.open(io.BytesIO(raw), "rb") as w:
            n, ch, width, sr = w.getnframes(), w.getnchannels(), w.getsampwidth(), w.getframerate()
            buf = w.readframes(n)
        dt = {1: "uint8", 2: "int16", 4: "int32"}[width]
        a = numpy.frombuffer(buf, dtype=dt).astype("float32")
        a = (a - 128.0) / 128.0 if width == 1 else a / float(2 ** (8 * width - 1))
        return (a.reshape(-1, ch) if ch > 1 else a), sr
    try:
        import soundfile
    except ImportError as exc:
        raise ImportError("decoding %r needs the soundfile package, which is not installed (wav files work without it): %s" % (name, exc))
    a, sr = soundfile.read(io.BytesIO(raw), dtype="float32")
    return a, sr


class OggZipDataset(CachedDataset2):
    """audio + text from zip files"""

    def __init__(self, path: Union[str, Sequence[str]], audio: Optional[Dict[str, Any]], targets: Optional[Union[Dict[str, Any], Vocabulary]],
                 targets_post_process=None, use_cache_manager: bool = False, segment_file: Optional[str] = None, zip_audio_files_have_name_as_prefix: bool = True,
                 fixed_random_subset: Optional[Union[float, int]] = None, fixed_random_subset_seed: int = 42, epoch_wise_filter: Optional[Dict] = None, **kwargs):
        super().__init__(**kwargs)
        self.paths = [path] if isinstance(path, str) else list(path)
        self._zips: Dict[str, zipfile.ZipFile] = {}
        self._prefix = zip_audio_files_have_name_as_prefix
        self.targets: Optional[Vocabulary] = None
        if targets is not None:
            self.targets = targets if isinstance(targets, Vocabulary) else Vocabulary.create_vocab(**targets)
            self.labels["classes"] = list(self.targets.labels)
        self.targets_post_process = targets_post_process
        self.feature_extractor = ExtractAudioFeatures(random_state=numpy.random.RandomState(1), **audio) if audio is not None else None
        self.num_inputs = self.feature_extractor.get_feature_dimension() if self.feature_extractor else 0
        self.num_outputs = {"raw": {"dtype": "string", "shape": ()}, "orth": (256, 1)}
        if self.feature_extractor:
            self.num_outputs["data"] = (self.num_inputs, 2)
        if self.targets:
            self.num_outputs["classes"] = (self.targets.num_labels, 1)
        self._data: List[Dict[str, Any]] = []
        for p in self.paths:
            self._data.extend(self._read_index(p))
        if segment_file:
            keep = set(line.strip() for line in open(segment_file) if line.strip())
            self._data = [d for d in self._data if self._tag(d) in keep]
        if fixed_random_subset:
            n = int(fixed_random_subset * len(self._data)) if isinstance(fixed_random_subset, float) else int(fixed_random_subset)
            rnd = numpy.random.RandomState(fixed_random_subset_seed)
            idx = list(range(len(self._data)))
            rnd.shuffle(idx)
            self._data = [self._data[i] for i in sorted(idx[:n])]
        from .meta import EpochWiseFilter

        self.epoch_wise_filter = EpochWiseFilter(epoch_wise_filter) if epoch_wise_filter else None
        self._order: List[int] = []

    def _read_index(self, path: str) -> List[Dict[str, Any]]:
        if os.path.isdir(path):
            name = os.path.basename(path.rstrip("/"))
            txt = open(os.path.join(path, name + ".txt")).read()
            entries = ast.literal_eval(txt)
            for e in entries:
                e["_src"] = ("dir", path, name)
            return entries
        zf = zipfile.ZipFile(path)
        self._zips[path] = zf
        name = os.path.splitext(os.path.basename(path))[0]
        txt_name = next(n for n in zf.namelist() if n.endswith(name + ".txt") or n == name + ".txt")
        entries = ast.literal_eval(zf.read(txt_name).decode("utf8"))
        for e in entries:
            e["_src"] = ("zip", path, name)
        return entries

    @staticmethod
    def _tag(d: Dict[str, Any]) -> str:
        return d.get("seq_name") or d["file"]

    def _read_bytes(self, d: Dict[str, Any]) -> bytes:
        kind, path, name = d["_src"]
        rel = ("%s/%s" % (name, d["file"])) if self._prefix else d["file"]
        if kind == "dir":
            fn = os.path.join(path, d["file"]) if not self._prefix else os.path.join(os.path.dirname(path.rstrip("/")), rel)
            if not os.path.exists(fn):
                fn = os.path.join(path, d["file"])
            return open(fn, "rb").read()
        return self._zips[path].read(rel)

    def __getstate__(self):
        s = dict(self.__dict__)
        s["_zips"] = {}
        return s

    def _dur(self, i: int) -> float:
        d = self._data[i]
        return float(d.get("duration") or len(d.get("text", "")))

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if not self._zips:
            for p in self.paths:
                if not os.path.isdir(p):
                    self._zips[p] = zipfile.ZipFile(p)
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            idx = {self._tag(d): i for i, d in enumerate(self._data)}
            self._order = [idx[t] for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self._data), get_seq_len=lambda i: int(self._dur(i) * 100)))
            if self.epoch_wise_filter:
                self._order = self.epoch_wise_filter.filter(epoch=epoch, seq_order=self._order, get_seq_len=lambda i: int(self._dur(i) * 100))
        if self.feature_extractor:
            self.feature_extractor.random_state = numpy.random.RandomState(self._get_random_seed_for_epoch(epoch=epoch))
        self._num_seqs = len(self._order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    def get_current_seq_order(self):
        return list(self._order)

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._data)

    def get_all_tags(self):
        return [self._tag(d) for d in self._data]

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        d = self._data[self._order[seq_idx]]
        tag = self._tag(d)
        feats: Dict[str, numpy.ndarray] = {}
        if self.feature_extractor:
            audio, sr = read_audio(self._read_bytes(d), d["file"])
            feats["data"] = self.feature_extractor.get_audio_features(audio, sr, seq_name=tag)
        text = d.get("text", "")
        if self.targets_post_process:
            text = self.targets_post_process(text)
        if self.targets:
            feats["classes"] = numpy.array(self.targets.get_seq(text), dtype="int32")
        feats["raw"] = numpy.array(text, dtype=object)
        feats["orth"] = numpy.frombuffer(text.encode("utf8"), dtype="uint8").copy()
        return DatasetSeq(seq_idx=seq_idx, seq_tag=tag, features=feats)

    def get_data_keys(self):
        return [k for k in ("data", "classes", "raw", "orth") if k in self.num_outputs]

    def get_target_list(self):
        return [k for k in ("classes", "raw", "orth") if k in self.num_outputs]

    def get_data_dtype(self, key):
        return {"data": "float32", "classes": "int32", "raw": "string", "orth": "uint8"}[key]

    def is_data_sparse(self, key):
        return key in ("classes", "orth")

    def get_data_dim(self, key):
        return {"data": self.num_inputs, "classes": self.targets.num_labels if self.targets else 0, "raw": 0, "orth": 256}[key]

    def get_data_shape(self, key):
        return [self.num_inputs] if key == "data" else []
