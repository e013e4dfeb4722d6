"""
Datasets over well-known corpora in their distribution formats: :class:`LibriSpeechCorpus` (directory or zip files of
``*.flac`` / ``*.wav`` + ``*.trans.txt``), :class:`TimitDataset` (``*.WAV`` + ``*.PHN``), :class:`BlissDataset` (Bliss XML
corpus), :class:`Enwik8Corpus` (byte-level language modelling on enwik8). Audio features are extracted on the fly with
:class:`~returnn_b200.datasets.util.feature_extraction.ExtractAudioFeatures`; ``.wav`` is decoded with the standard library,
``.flac`` / ``.ogg`` / NIST sphere need the ``soundfile`` package.

Reference: returnn/datasets/generating.py (TimitDataset :1280, BlissDataset :1865, LibriSpeechCorpus :1996, Enwik8Corpus :2401).
These classes are also importable from :mod:`returnn_b200.datasets.generating`, where the reference has them.
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union
import glob as _glob
import os
import re
import zipfile
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from .util.vocabulary import Vocabulary, BytePairEncoding, CharacterTargets
from .util.feature_extraction import ExtractAudioFeatures
from ..log import log


def _subset_indices(n: int, fixed_random_subset: Optional[Union[float, int]], seed: int = 42) -> List[int]:
    """a deterministic random subset of range(n), in corpus order"""
    if not fixed_random_subset:
        return list(range(n))
    k = int(fixed_random_subset * n) if isinstance(fixed_random_subset, float) and fixed_random_subset <= 1 else int(fixed_random_subset)
    assert 0 < k <= n, "fixed_random_subset %r of %i sequences" % (fixed_random_subset, n)
    idx = list(range(n))
    numpy.random.RandomState(seed).shuffle(idx)
    return sorted(idx[:k])


def _make_targets(targets, bpe, chars) -> Optional[Vocabulary]:
    if isinstance(targets, dict):
        assert bpe is None and chars is None
        return Vocabulary.create_vocab(**targets)
    if targets == "bpe" or (targets is None and bpe is not None):
        assert bpe is not None and chars is None
        return BytePairEncoding(**bpe)
    if targets == "chars" or (targets is None and chars is not None):
        assert bpe is None and chars is not None
        return CharacterTargets(**chars)
    if targets is None:
        return None
    raise ValueError("invalid targets %r: give a vocabulary dict, 'bpe' or 'chars'" % (targets,))


class _AudioTextCorpus(CachedDataset2):
    """
    Shared part of the audio corpora: a list of entries (each knows how to load its audio and has a transcription), an optional
    vocabulary for ``classes``, feature extraction for ``data``, ordering by duration / length, ``epoch_wise_filter``.
    """

    def __init__(self, *, audio: Optional[Dict[str, Any]], targets: Optional[Vocabulary], orth_post_process=None,
                 fixed_random_subset=None, epoch_wise_filter: Optional[Dict] = None, **kwargs):
        super().__init__(**kwargs)
        self.targets = targets
        if targets is not None:
            self.labels["classes"] = list(targets.labels)
        self.orth_post_process = None
        if orth_post_process:
            from .lm import get_post_processor_function

            self.orth_post_process = get_post_processor_function(orth_post_process)
        self._audio_random = numpy.random.RandomState(1)
        self.feature_extractor = ExtractAudioFeatures(random_state=self._audio_random, **audio) if audio is not None else None
        self.num_inputs = self.feature_extractor.get_feature_dimension() if self.feature_extractor else 0
        self.num_outputs = {"raw": {"dtype": "string", "shape": ()}, "orth": (256, 1)}
        if self.feature_extractor:
            self.num_outputs["data"] = (self.num_inputs, 2)
        if self.targets is not None:
            self.num_outputs["classes"] = (self.targets.num_labels, 1)
        self._entries: List[Dict[str, Any]] = []
        self._fixed_random_subset = fixed_random_subset
        from .meta import EpochWiseFilter

        self.epoch_wise_filter = EpochWiseFilter(epoch_wise_filter) if epoch_wise_filter else None
        self._order: List[int] = []

    def _finish_entries(self):
        keep = _subset_indices(len(self._entries), self._fixed_random_subset)
        self._entries = [self._entries[i] for i in keep]

    # -- per entry, from the subclass
    def _load_audio(self, entry: Dict[str, Any]) -> Tuple[numpy.ndarray, int]:
        raise NotImplementedError

    def _entry_len(self, i: int) -> int:
        """a cheap length for the length-based orderings: characters of the transcription"""
        return len(self._entries[i]["text"])

    # -- Dataset API
    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._entries)

    def get_all_tags(self) -> List[str]:
        return [e["tag"] for e in self._entries]

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if epoch is not None:
            self._audio_random.seed(self._get_random_seed_for_epoch(epoch))
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            by_tag = {e["tag"]: i for i, e in enumerate(self._entries)}
            self._order = [by_tag[t] for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self._entries), get_seq_len=self._entry_len))
            if self.epoch_wise_filter is not None and epoch is not None:
                self._order = list(self.epoch_wise_filter.filter(epoch=epoch, seq_order=self._order, get_seq_len=self._entry_len))
        self._num_seqs = len(self._order)
        return True

    @property
    def num_seqs(self) -> int:
        return len(self._order)

    def supports_seq_order_sorting(self) -> bool:
        return True

    def get_current_seq_order(self):
        return list(self._order)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        entry = self._entries[self._order[seq_idx]]
        feats: Dict[str, numpy.ndarray] = {}
        if self.feature_extractor is not None:
            audio, sample_rate = self._load_audio(entry)
            feats["data"] = self.feature_extractor.get_audio_features(audio, sample_rate, seq_name=entry["tag"])
        text = entry["text"]
        if self.orth_post_process:
            text = self.orth_post_process(text)
        if self.targets is not None:
            feats["classes"] = numpy.array(self.targets.get_seq(text), dtype="int32")
        feats["raw"] = numpy.array(text, dtype=object)
        feats["orth"] = numpy.frombuffer(text.encode("utf8"), dtype="uint8").copy()
        return DatasetSeq(seq_idx=seq_idx, seq_tag=entry["tag"], features=feats)

    def get_data_keys(self):
        return [k for k in ("data", "classes", "raw", "orth") if k in self.num_outputs]

    def get_target_list(self):
        return [k for k in ("classes", "raw", "orth") if k in self.num_outputs]

    def get_data_dtype(self, key):
        return {"data": "float32", "classes": "int32", "raw": "string", "orth": "uint8"}[key]

    def is_data_sparse(self, key):
        return key in ("classes", "orth")

    def get_data_dim(self, key):
        if key == "raw":
            return 0
        return self.num_outputs[key][0]

    def get_data_shape(self, key):
        return [self.num_inputs] if key == "data" else []


class LibriSpeechCorpus(_AudioTextCorpus):
    """
    LibriSpeech (https://www.openslr.org/12/). ``path`` contains ``<subset>/<speaker>/<chapter>/*.flac`` with one
    ``<speaker>-<chapter>.trans.txt`` per chapter (lines ``<speaker>-<chapter>-<seq> TRANSCRIPTION``), or with ``use_zip`` one
    ``<subset>.zip`` per subset with the same tree inside. ``prefix`` selects the subsets: ``"train"``, ``"dev"``, ``"dev-other"``,
    ``"train-clean-100"``, ...  Keys: ``data`` (features), ``classes`` (``targets`` / ``bpe`` / ``chars``), ``raw``, ``orth``.
    """

    def __init__(self, path: str, prefix: str, audio: Optional[Dict[str, Any]], orth_post_process=None, targets=None, chars=None, bpe=None,
                 use_zip: bool = False, use_ogg: bool = False, use_cache_manager: bool = False, fixed_random_subset=None,
                 epoch_wise_filter=None, name: Optional[str] = None, seq_tag_format: str = "%(subdir)s-%(speaker)i-%(chapter)i-%(seq)04i", **kwargs):
        assert prefix.split("-")[0] in ("train", "dev", "test"), "LibriSpeechCorpus: prefix %r" % (prefix,)
        super().__init__(audio=audio, targets=_make_targets(targets, bpe, chars), orth_post_process=orth_post_process,
                         fixed_random_subset=fixed_random_subset, epoch_wise_filter=epoch_wise_filter, name=name or ("prefix:" + prefix), **kwargs)
        self.path, self.prefix, self.use_zip, self.use_ogg = path, prefix, use_zip, use_ogg
        self._seq_tag_format = seq_tag_format
        self._zip_files: Dict[str, zipfile.ZipFile] = {}
        if use_zip:
            fns = sorted(_glob.glob("%s/%s*.zip" % (path, prefix)))
            assert fns, "LibriSpeechCorpus: no zip files %s/%s*.zip" % (path, prefix)
            if use_cache_manager:
                from ..utils.basic import cf

                fns = [cf(fn) for fn in fns]
            self._zip_files = {os.path.splitext(os.path.basename(fn))[0]: zipfile.ZipFile(fn) for fn in fns}
        self._collect_entries()
        self._finish_entries()

    _TRANS_RE = re.compile(r"^(\d+)-(\d+)\.trans\.txt$")

    def _add_transcriptions(self, subdir: str, speaker: int, chapter: int, lines: Sequence[str]):
        for line in lines:
            line = line.strip()
            if not line:
                continue
            seq_name, _, text = line.partition(" ")
            sp, ch, seq = (int(x) for x in seq_name.split("-"))
            assert (sp, ch) == (speaker, chapter), "unexpected utterance %r in the transcriptions of %i-%i" % (seq_name, speaker, chapter)
            fields = {"subdir": subdir, "speaker": speaker, "chapter": chapter, "seq": seq}
            self._entries.append(dict(fields, text=text, tag=self._seq_tag_format % fields))

    def _collect_entries(self):
        if self.use_zip:
            for subdir, zf in sorted(self._zip_files.items()):
                for info in sorted(zf.infolist(), key=lambda i: i.filename):
                    m = self._TRANS_RE.match(os.path.basename(info.filename))
                    if m:
                        self._add_transcriptions(subdir, int(m.group(1)), int(m.group(2)), zf.read(info).decode("utf8").splitlines())
        else:
            for subdir_path in sorted(_glob.glob("%s/%s*" % (self.path, self.prefix))):
                if not os.path.isdir(subdir_path):
                    continue
                subdir = os.path.basename(subdir_path)
                for fn in sorted(_glob.glob("%s/*/*/*.trans.txt" % subdir_path)):
                    m = self._TRANS_RE.match(os.path.basename(fn))
                    assert m, fn
                    with open(fn, encoding="utf8") as f:
                        self._add_transcriptions(subdir, int(m.group(1)), int(m.group(2)), f.readlines())
        assert self._entries, "LibriSpeechCorpus: nothing found under %s for prefix %r" % (self.path, self.prefix)

    def _audio_candidates(self, e: Dict[str, Any]) -> List[str]:
        stem = "%(subdir)s/%(speaker)i/%(chapter)i/%(speaker)i-%(chapter)i-%(seq)04i" % e
        exts = [".flac.ogg", ".ogg"] if self.use_ogg else [".flac", ".wav"]
        return [stem + x for x in exts]

    def _load_audio(self, entry):
        from .audio import read_audio

        for rel in self._audio_candidates(entry):
            if self.use_zip:
                zf = self._zip_files[entry["subdir"]]
                for name in (rel, "LibriSpeech/" + rel):
                    if name in zf.namelist():
                        return read_audio(zf.read(name), name)
            else:
                fn = os.path.join(self.path, rel)
                if os.path.exists(fn):
                    with open(fn, "rb") as f:
                        return read_audio(f.read(), fn)
        raise FileNotFoundError("LibriSpeechCorpus: no audio file for %s (tried %s)" % (entry["tag"], self._audio_candidates(entry)))

    def __getstate__(self):
        st = dict(self.__dict__)
        st["_zip_files"] = {}
        return st

    def __setstate__(self, st):
        self.__dict__.update(st)
        if self.use_zip:
            fns = sorted(_glob.glob("%s/%s*.zip" % (self.path, self.prefix)))
            self._zip_files = {os.path.splitext(os.path.basename(fn))[0]: zipfile.ZipFile(fn) for fn in fns}


class TimitDataset(_AudioTextCorpus):
    """
    DARPA TIMIT: ``<timit_dir>/{train,test}/<dialect>/<speaker>/<utterance>.{wav,phn}``. ``classes`` are frame-wise phone labels
    derived from the ``.phn`` segmentation (sample ranges), over the 61 phones folded to ``num_phones`` in (61, 48, 39);
    ``data`` are MFCC (or other) features at ``feature_step_len``. ``train=True`` takes ``train/`` without the ``sa`` sentences,
    as is customary; ``demo_play_audio`` and preloading are not offered here.
    """

    Phones61 = ("aa ae ah ao aw ax ax-h axr ay b bcl ch d dcl dh dx eh el em en eng epi er ey f g gcl h# hh hv ih ix iy jh k kcl l m n "
                "ng nx ow oy p pau pcl q r s sh t tcl th uh uw ux v w y z zh").split()
    # folding 61 -> 48 -> 39 (Lee & Hon 1989)
    _Fold48 = {"ux": "uw", "axr": "er", "em": "m", "nx": "n", "eng": "ng", "hv": "hh", "pcl": "cl", "tcl": "cl", "kcl": "cl", "qcl": "cl",
               "bcl": "vcl", "dcl": "vcl", "gcl": "vcl", "h#": "sil", "pau": "sil", "#h": "sil", "ax-h": "ax", "q": None}
    _Fold39 = {"ao": "aa", "ax": "ah", "ix": "ih", "el": "l", "en": "n", "zh": "sh", "cl": "sil", "vcl": "sil", "epi": "sil"}

    def __init__(self, timit_dir: str, train: bool = True, preload: bool = False, features: str = "mfcc", num_feature_filters: int = 40,
                 feature_window_len: float = 0.025, feature_step_len: float = 0.010, with_delta: Union[bool, int] = False,
                 norm_mean=None, norm_std_dev=None, random_permute_audio=None, num_phones: int = 61, demo_play_audio: bool = False,
                 fixed_random_seed: Optional[int] = None, **kwargs):
        assert num_phones in (61, 48, 39)
        assert not demo_play_audio, "TimitDataset: audio playback is not available"
        audio = dict(features=features, num_feature_filters=num_feature_filters, window_len=feature_window_len, step_len=feature_step_len,
                     with_delta=with_delta, norm_mean=norm_mean, norm_std_dev=norm_std_dev, random_permute=random_permute_audio)
        super().__init__(audio=audio, targets=None, fixed_random_seed=fixed_random_seed, **kwargs)
        self._timit_dir = timit_dir
        self._is_train = train
        self._step_len = feature_step_len
        self._num_phones = num_phones
        self._phone_map, self.labels["classes"] = self._make_phone_map(num_phones)
        self.num_outputs = {"data": (self.num_inputs, 2), "classes": (len(self.labels["classes"]), 1)}
        self._collect_entries()
        assert self._entries, "%s: no utterances" % type(self).__name__
        self._finish_entries()

    def _collect_entries(self):
        """fills ``self._entries`` from ``<timit_dir>/{train,test}/<dialect>/<speaker>/<utterance>.{wav,phn}``"""
        timit_dir, train = self._timit_dir, self._is_train
        sub = "train" if train else "test"
        root = None
        for cand in (os.path.join(timit_dir, sub), os.path.join(timit_dir, sub.upper())):
            if os.path.isdir(cand):
                root = cand
        assert root, "TimitDataset: %s has no %s directory" % (timit_dir, sub)
        for phn in sorted(_glob.glob(root + "/*/*/*.[pP][hH][nN]")):
            base = os.path.splitext(phn)[0]
            utt = os.path.basename(base).lower()
            if train and utt.startswith("sa"):
                continue  # the two dialect sentences that every speaker reads
            wav = next((base + e for e in (".wav", ".WAV") if os.path.exists(base + e)), None)
            if wav is None:
                continue
            rel = os.path.relpath(base, root).replace(os.sep, "/").lower()
            self._entries.append({"tag": "%s/%s" % (sub, rel), "phn": phn, "wav": wav, "text": ""})

    @classmethod
    def _make_phone_map(cls, num_phones: int) -> Tuple[Dict[str, Optional[str]], List[str]]:
        mapping: Dict[str, Optional[str]] = {}
        for p in cls.Phones61:
            q: Optional[str] = p
            if num_phones <= 48:
                q = cls._Fold48.get(p, p)
            if num_phones <= 39 and q is not None:
                q = cls._Fold39.get(q, q)
            mapping[p] = q
        labels = sorted({q for q in mapping.values() if q is not None})
        return mapping, labels

    def _entry_len(self, i: int) -> int:
        return os.path.getsize(self._entries[i]["wav"])

    def _load_audio(self, entry):
        from .audio import read_audio

        with open(entry["wav"], "rb") as f:
            raw = f.read()
        name = entry["wav"]
        if raw[:4] != b"RIFF":
            name = name + ".nist"  # NIST sphere header: needs soundfile
        else:
            name = os.path.splitext(name)[0] + ".wav"
        return read_audio(raw, name)

    def _frame_labels(self, entry, num_frames: int, sample_rate: int) -> numpy.ndarray:
        label_idx = {p: i for i, p in enumerate(self.labels["classes"])}
        out = numpy.zeros((num_frames,), dtype="int32")
        sil = label_idx.get("sil", label_idx.get("h#", 0))
        out[:] = sil
        with open(entry["phn"]) as f:
            for line in f:
                parts = line.split()
                if len(parts) != 3:
                    continue
                start, end, phone = int(parts[0]), int(parts[1]), parts[2].lower()
                mapped = self._phone_map.get(phone, phone)
                if mapped is None:
                    continue  # glottal stop: dropped by the folding, the frames keep the neighbouring label
                f0 = int(round(start / sample_rate / self._step_len))
                f1 = int(round(end / sample_rate / self._step_len))
                out[f0: max(f1, f0 + 1)] = label_idx[mapped]
        return out

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        entry = self._entries[self._order[seq_idx]]
        audio, sample_rate = self._load_audio(entry)
        feats = self.feature_extractor.get_audio_features(audio, sample_rate, seq_name=entry["tag"])
        return DatasetSeq(seq_idx=seq_idx, seq_tag=entry["tag"], features={"data": feats, "classes": self._frame_labels(entry, feats.shape[0], sample_rate)})

    def get_data_keys(self):
        return ["data", "classes"]

    def get_target_list(self):
        return ["classes"]


class NltkTimitDataset(TimitDataset):
    """
    The TIMIT sample that NLTK distributes (160 training utterances, no test set): ``<nltk data>/corpora/timit/<dialect>-<speaker>/<utterance>.{wav,phn}``.
    ``nltk_download_dir`` names the NLTK data directory; without it the directories NLTK itself would search are tried (``NLTK_DATA``,
    ``~/nltk_data``, ``/usr/share/nltk_data`` ...). Nothing is downloaded here. The one set is split 90 / 10 into ``train=True`` / ``train=False``.
    Parity: returnn/datasets/generating.py:1800.
    """

    def __init__(self, nltk_download_dir: Optional[str] = None, **kwargs):
        self._nltk_download_dir = nltk_download_dir
        super().__init__(timit_dir=self._find_dir(nltk_download_dir), **kwargs)

    @staticmethod
    def _find_dir(nltk_download_dir: Optional[str]) -> str:
        cands = [nltk_download_dir] if nltk_download_dir else []
        if not cands:
            cands += [p for p in os.environ.get("NLTK_DATA", "").split(os.pathsep) if p]
            try:
                import nltk.data  # noqa

                cands += list(nltk.data.path)
            except ImportError:
                pass
            cands += [os.path.expanduser("~/nltk_data"), "/usr/share/nltk_data", "/usr/local/share/nltk_data", "/usr/lib/nltk_data"]
        for c in cands:
            d = os.path.join(c, "corpora", "timit")
            if os.path.isdir(d):
                return d
        raise FileNotFoundError("NltkTimitDataset: no corpora/timit under %s (fetch it with nltk.download('timit') and pass nltk_download_dir)" % cands)

    def _collect_entries(self):
        entries = []
        for phn in sorted(_glob.glob(self._timit_dir + "/*/*.[pP][hH][nN]")):
            base = os.path.splitext(phn)[0]
            wav = next((base + e for e in (".wav", ".WAV") if os.path.exists(base + e)), None)
            if wav is None:
                continue
            rel = os.path.relpath(base, self._timit_dir).replace(os.sep, "/").lower()
            entries.append({"tag": rel, "phn": phn, "wav": wav, "text": ""})
        split = int(len(entries) * 0.9)
        self._entries.extend(entries[:split] if self._is_train else entries[split:])


class BlissDataset(_AudioTextCorpus):
    """
    Bliss XML corpus (``<corpus><recording audio=...><segment name= start= end=><orth>...``, optionally gzipped, with
    ``<include file=...>``): one sequence per segment, features from the segment's part of the recording, ``classes`` from
    ``vocab_file`` (a Python dict ``{label: index}``) with BPE merges from ``bpe_file``, or characters when no BPE file is given.
    """

    def __init__(self, path: str, vocab_file: str, bpe_file: Optional[str] = None, num_feature_filters: int = 40,
                 feature_window_len: float = 0.025, feature_step_len: float = 0.010, with_delta: Union[bool, int] = False,
                 norm_mean=None, norm_std_dev=None, **kwargs):
        if bpe_file:
            vocab: Vocabulary = BytePairEncoding(vocab_file=vocab_file, bpe_file=bpe_file, seq_postfix=None, unknown_label=None)
        else:
            vocab = Vocabulary(vocab_file=vocab_file, unknown_label=None)
        audio = dict(num_feature_filters=num_feature_filters, window_len=feature_window_len, step_len=feature_step_len, with_delta=with_delta,
                     norm_mean=norm_mean, norm_std_dev=norm_std_dev)
        super().__init__(audio=audio, targets=vocab, **kwargs)
        self._word_level = bool(bpe_file)
        self.path = path
        self._parse(path)
        assert self._entries, "BlissDataset: no segments in %s" % path
        self._finish_entries()

    def _parse(self, path: str, prefix: str = ""):
        import gzip
        import xml.etree.ElementTree as ET

        opener = gzip.open if path.endswith(".gz") else open
        with opener(path, "rb") as f:
            root = ET.parse(f).getroot()
        name = root.attrib.get("name", "")
        corpus_prefix = (prefix + name + "/") if name else prefix
        for node in root:
            if node.tag == "include":
                self._parse(os.path.join(os.path.dirname(path), node.attrib["file"]), corpus_prefix)
            elif node.tag == "recording":
                audio_fn = node.attrib.get("audio", "")
                if audio_fn and not os.path.isabs(audio_fn):
                    audio_fn = os.path.join(os.path.dirname(path), audio_fn)
                rec_name = node.attrib.get("name", "")
                for seg in node.iter("segment"):
                    orth = seg.find("orth")
                    text = " ".join((orth.text or "").split()) if orth is not None else ""
                    self._entries.append({"tag": "%s%s/%s" % (corpus_prefix, rec_name, seg.attrib.get("name", str(len(self._entries) + 1))),
                                          "audio": audio_fn, "start": float(seg.attrib.get("start", 0.0)),
                                          "end": float(seg.attrib["end"]) if "end" in seg.attrib else None, "text": text})

    def _entry_len(self, i: int) -> int:
        e = self._entries[i]
        return int(1000 * (e["end"] - e["start"])) if e["end"] is not None else len(e["text"])

    def _load_audio(self, entry):
        from .audio import read_audio

        with open(entry["audio"], "rb") as f:
            audio, sample_rate = read_audio(f.read(), entry["audio"])
        i0 = int(entry["start"] * sample_rate)
        i1 = int(entry["end"] * sample_rate) if entry["end"] is not None else len(audio)
        return audio[i0:i1], sample_rate


class Enwik8Corpus(CachedDataset2):
    """
    Byte-level language modelling on enwik8 (the first 10^8 bytes of an English Wikipedia dump): ``path`` holds ``enwik8.zip`` (member
    ``enwik8``) or the prepared ``enwik8.hdf5``; the last 2 x 5M bytes are validation and test. A sequence is ``seq_len`` bytes of
    the subset, ``data`` the bytes (as indices into the used byte values) and ``classes`` the same shifted by one.
    ``batch_num_seqs``: order the sequences so that, batched in groups of that size, every batch entry continues where it was in the
    previous batch (hidden state can be carried over). The archive is not downloaded: this framework runs without network access.
    """

    _hdf_cache: Dict[str, Any] = {}

    def __init__(self, path: str, subset: str, seq_len: int, batch_num_seqs: Optional[int] = None, subsubset=None, **kwargs):
        assert subset in ("training", "validation", "test")
        super().__init__(**kwargs)
        assert os.path.isdir(path), "Enwik8Corpus: %s is not a directory" % path
        self.path = path
        f = self._prepare()
        self._unique = numpy.asarray(f.attrs["unique"])
        labels = [bytes([int(b)]) for b in self._unique]
        self.labels = {"data": labels, "classes": labels}
        self.num_inputs = len(labels)
        self.num_outputs = {"data": [self.num_inputs, 1], "classes": [self.num_inputs, 1]}
        data = f["split/%s/default" % subset]
        if subsubset:
            data = data[:subsubset] if isinstance(subsubset, int) else data[subsubset[0]: subsubset[1]]
        else:
            data = data[...]
        self._data = numpy.asarray(data, dtype="uint8")
        assert len(self._data) > 1
        self._seq_len = seq_len
        self._batch_num_seqs = batch_num_seqs
        self._seq_starts = numpy.arange(0, len(self._data) - 1, seq_len)
        self._seq_order: Sequence[int] = []

    @property
    def _hdf_filename(self) -> str:
        return self.path + "/enwik8.hdf5"

    @property
    def _zip_filename(self) -> str:
        return self.path + "/enwik8.zip"

    def _prepare(self):
        fn = self._hdf_filename
        if fn in self._hdf_cache:
            return self._hdf_cache[fn]
        from ..utils.h5_shim import get_h5py

        h5py = get_h5py()
        if not os.path.exists(fn):
            if not os.path.exists(self._zip_filename):
                raise FileNotFoundError("Enwik8Corpus: neither %s nor %s exists (get enwik8.zip from mattmahoney.net/dc/ and put it there)" % (fn, self._zip_filename))
            print("%s: create %s" % (self, fn), file=log.v2)
            raw = numpy.frombuffer(zipfile.ZipFile(self._zip_filename).read("enwik8"), dtype=numpy.uint8)
            unique, data = numpy.unique(raw, return_inverse=True)
            data = data.astype("uint8")
            n_test = min(5000000, len(data) // 10)
            out = h5py.File(fn, "w")
            out.attrs["unique"] = unique
            split = out.create_group("split")
            for name, part in (("training", data[: -2 * n_test]), ("validation", data[-2 * n_test: -n_test]), ("test", data[-n_test:])):
                split.create_group(name).create_dataset("default", data=part, compression="gzip")
            out.close()
        self._hdf_cache[fn] = h5py.File(fn, "r")
        return self._hdf_cache[fn]

    def get_data_dtype(self, key):
        return "uint8"

    def supports_sharding(self) -> bool:
        return self._batch_num_seqs is None

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        n = len(self._seq_starts)
        if self._batch_num_seqs is None:
            self._seq_order = list(self.get_seq_order_for_epoch(epoch=epoch or 1, num_seqs=n, get_seq_len=lambda _i: self._seq_len))
        else:
            part = None
            if self.partition_epoch and self.partition_epoch > 1 and epoch is not None:
                part = (epoch - 1) % self.partition_epoch
            n -= n % self._batch_num_seqs
            assert n > 0
            # row b of the [batch_num_seqs, n / batch_num_seqs] grid is one contiguous stretch of text; reading the grid column by column
            # puts consecutive pieces of every stretch at the same position of consecutive batches
            order = numpy.arange(n).reshape(self._batch_num_seqs, n // self._batch_num_seqs).transpose().flatten()
            if part is not None:
                sizes = [n // self.partition_epoch + (1 if i < n % self.partition_epoch else 0) for i in range(self.partition_epoch)]
                start = sum(sizes[:part])
                order = order[start: start + sizes[part]]
            self._seq_order = [int(i) for i in order]
        self._num_seqs = len(self._seq_order)
        self._num_timesteps = len(self._data) - 1
        return True

    @property
    def num_seqs(self) -> int:
        return len(self._seq_order)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._seq_order):
            return None
        start = int(self._seq_starts[self._seq_order[seq_idx]])
        end = min(start + 1 + self._seq_len, len(self._data))
        data = numpy.array(self._data[start:end], dtype="uint8")
        return DatasetSeq(seq_idx=seq_idx, features=data[:-1], targets=data[1:], seq_tag="offset_%i_%i" % (start, len(data) - 1))
