"""
Text datasets (reference: returnn/datasets/lm.py): :class:`LmDataset` (one sentence per line, optionally gzipped, turned
into label sequences by a vocabulary / orthography symbols), :class:`TranslationDataset` (parallel source / target text
files), :class:`Lexicon` (Bliss XML lexicon) and :class:`PhoneSeqGenerator`.
"""

from __future__ import annotations
from typing import Tuple, Any, Callable, Dict, Iterator, List, Optional, Sequence, Union
import gzip
import re
import os
import xml.etree.ElementTree as ElementTree
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2
from .util.vocabulary import Vocabulary


def _open_text(filename: str):
    if filename.endswith(".gz"):
        return gzip.open(filename, "rt", encoding="utf8")
    return open(filename, "rt", encoding="utf8")


def read_corpus(filename: str, skip_empty_lines: bool = True, decode: bool = True, out_list: Optional[List[str]] = None) -> List[str]:
    """all lines of a text file (or the ``<orth>`` elements of a Bliss corpus XML)"""
    out = out_list if out_list is not None else []
    if filename.endswith(".xml") or filename.endswith(".xml.gz"):
        iter_corpus(filename, skip_empty_lines=skip_empty_lines, callback=out.append)
        return out
    with _open_text(filename) as f:
        for line in f:
            line = line.rstrip("\n")
            if skip_empty_lines and not line.strip():
                continue
            out.append(line)
    return out


def iter_corpus(filename: str, callback: Callable[[str], None], skip_empty_lines: bool = True, decode: bool = True):
    """call ``callback(orth)`` for every sentence"""
    if filename.endswith(".xml") or filename.endswith(".xml.gz"):
        with (gzip.open(filename, "rb") if filename.endswith(".gz") else open(filename, "rb")) as f:
            for _, elem in ElementTree.iterparse(f, events=("end",)):
                if elem.tag == "orth":
                    text = (elem.text or "").strip()
                    if text or not skip_empty_lines:
                        callback(text)
                    elem.clear()
        return
    for line in read_corpus(filename, skip_empty_lines=skip_empty_lines):
        callback(line)


class LmDataset(CachedDataset2):
    """
    Language-model data: every line is one sequence; ``data`` are the label indices (with optional ``seq_end_symbol`` /
    ``auto_replace_unknown_symbol``), ``delayed`` the same shifted right by ``delayed_seq_data_start_symbol``.
    """

    def __init__(self, corpus_file: Union[str, Sequence[str], Callable[[], Sequence[str]]], orth_vocab: Optional[Union[Dict[str, Any], Vocabulary]] = None,
                 orth_symbols_file: Optional[str] = None, orth_symbols_map_file: Optional[str] = None, orth_replace_map_file: Optional[str] = None,
                 word_based: bool = False, word_end_symbol: Optional[str] = None, seq_end_symbol: Optional[str] = "[END]",
                 unknown_symbol: Optional[str] = "[UNKNOWN]", parse_orth_opts: Optional[Dict[str, Any]] = None, phone_info: Optional[Dict[str, Any]] = None,
                 add_random_phone_seqs: int = 0, auto_replace_unknown_symbol: bool = False, log_auto_replace_unknown_symbols: int = 10,
                 log_skipped_seqs: int = 10, error_on_invalid_seq: bool = True, add_delayed_seq_data: bool = False,
                 delayed_seq_data_start_symbol: str = "[START]", dtype: Optional[str] = None, tag_prefix: Optional[str] = None, skip_empty_lines: bool = True,
                 use_cache_manager: bool = False, **kwargs):
        super().__init__(**kwargs)
        if callable(corpus_file):
            corpus_file = corpus_file()
        self._corpus_files = [corpus_file] if isinstance(corpus_file, str) else list(corpus_file)
        self.word_based = word_based
        self.word_end_symbol = word_end_symbol
        self.seq_end_symbol = seq_end_symbol
        self.unknown_symbol = unknown_symbol
        self.auto_replace_unknown_symbol = auto_replace_unknown_symbol
        self.error_on_invalid_seq = error_on_invalid_seq
        self.add_delayed_seq_data = add_delayed_seq_data
        self.delayed_seq_data_start_symbol = delayed_seq_data_start_symbol
        self.tag_prefix = tag_prefix or "line-"
        self.orth_vocab: Optional[Vocabulary] = None
        self.orth_symbols_map: Dict[str, int] = {}
        if orth_vocab is not None:
            self.orth_vocab = orth_vocab if isinstance(orth_vocab, Vocabulary) else Vocabulary.create_vocab(**orth_vocab)
            num_labels = self.orth_vocab.num_labels
            self.labels["data"] = list(self.orth_vocab.labels)
        else:
            if orth_symbols_map_file:
                for line in read_corpus(orth_symbols_map_file):
                    sym, idx = line.rsplit(None, 1)
                    self.orth_symbols_map[sym] = int(idx)
            elif orth_symbols_file:
                for i, line in enumerate(read_corpus(orth_symbols_file)):
                    self.orth_symbols_map[line.strip() if word_based else line.rstrip("\n")] = i
            else:
                raise ValueError("%s: need orth_vocab, orth_symbols_file or orth_symbols_map_file" % self)
            num_labels = max(self.orth_symbols_map.values()) + 1
            labels = [""] * num_labels
            for s, i in self.orth_symbols_map.items():
                labels[i] = s
            self.labels["data"] = labels
        if dtype is None:
            dtype = "int32" if num_labels > 255 else "uint8"
        self.dtype = dtype
        self.num_inputs = num_labels
        self.num_outputs = {"data": (num_labels, 1)}
        if add_delayed_seq_data:
            self.num_outputs["delayed"] = (num_labels, 1)
            self.labels["delayed"] = self.labels["data"]
        self.orths: List[str] = []
        for fn in self._corpus_files:
            read_corpus(fn, skip_empty_lines=skip_empty_lines, out_list=self.orths)
        self._order: List[int] = []
        self._num_unknown = 0

    def get_data_keys(self):
        return ["data"] + (["delayed"] if self.add_delayed_seq_data else [])

    def get_target_list(self):
        return ["delayed"] if self.add_delayed_seq_data else []

    def get_data_dtype(self, key):
        return self.dtype

    def is_data_sparse(self, key):
        return True

    def get_data_dim(self, key):
        return self.num_outputs[key][0]

    def get_data_shape(self, key):
        return []

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self.orths)

    def get_all_tags(self):
        return ["%s%i" % (self.tag_prefix, i) for i in range(len(self.orths))]

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            self._order = [int(t[len(self.tag_prefix):]) for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self.orths), get_seq_len=lambda i: len(self.orths[i])))
        self._num_seqs = len(self._order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    def get_current_seq_order(self):
        return list(self._order)

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def _encode(self, orth: str) -> Optional[List[int]]:
        if self.orth_vocab is not None:
            ids = list(self.orth_vocab.get_seq(orth))
            if self.seq_end_symbol and self.seq_end_symbol in getattr(self.orth_vocab, "_vocab", {}):
                ids.append(self.orth_vocab.label_to_id(self.seq_end_symbol))
            return ids
        syms = orth.split() if self.word_based else list(orth)
        if self.word_end_symbol and not self.word_based:
            syms = [self.word_end_symbol if s == " " else s for s in syms]
        if self.seq_end_symbol:
            syms.append(self.seq_end_symbol)
        ids = []
        for s in syms:
            if s in self.orth_symbols_map:
                ids.append(self.orth_symbols_map[s])
            elif self.auto_replace_unknown_symbol and self.unknown_symbol in self.orth_symbols_map:
                self._num_unknown += 1
                ids.append(self.orth_symbols_map[self.unknown_symbol])
            elif self.error_on_invalid_seq:
                raise ValueError("%s: symbol %r of %r is not in the symbol table" % (self, s, orth))
            else:
                return None
        return ids

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        while seq_idx < len(self._order):
            line = self._order[seq_idx]
            ids = self._encode(self.orths[line])
            if ids is None:
                # skipped sequences are replaced by an empty one to keep indices dense
                ids = []
            data = numpy.array(ids, dtype=self.dtype)
            feats = {"data": data}
            if self.add_delayed_seq_data:
                start = self.orth_symbols_map.get(self.delayed_seq_data_start_symbol, 0) if self.orth_vocab is None else \
                    self.orth_vocab.label_to_id(self.delayed_seq_data_start_symbol)
                feats["delayed"] = numpy.concatenate([numpy.array([start], dtype=self.dtype), data[:-1]])
            return DatasetSeq(seq_idx=seq_idx, seq_tag="%s%i" % (self.tag_prefix, line), features=feats)
        return None


class TranslationDataset(CachedDataset2):
    """
    Parallel text: ``<path>/source.<file_postfix>[.gz]`` and ``target.<file_postfix>[.gz]`` with one sentence per line and
    vocabularies ``source.vocab.pkl`` / ``target.vocab.pkl`` (pickled ``{symbol: index}``); keys ``data`` and ``classes``.
    """

    source_file_prefix = "source"
    target_file_prefix = "target"

    def __init__(self, path: str, file_postfix: str, source_postfix: str = "", target_postfix: str = "", source_only: bool = False,
                 search_without_reference: bool = False, unknown_label: Optional[Union[str, Dict[str, str]]] = None, seq_list_file: Optional[str] = None,
                 use_cache_manager: bool = False, **kwargs):
        super().__init__(**kwargs)
        import pickle

        self.path, self.file_postfix = path, file_postfix
        self.source_only = source_only or search_without_reference
        self._add = {"data": source_postfix, "classes": target_postfix}
        self._keys = ["data"] if self.source_only else ["data", "classes"]
        prefix = {"data": self.source_file_prefix, "classes": self.target_file_prefix}
        self._vocabs: Dict[str, Dict[str, int]] = {}
        self._lines: Dict[str, List[str]] = {}
        self._unknown: Dict[str, Optional[str]] = {}
        for k in self._keys:
            vfile = os.path.join(path, "%s.vocab.pkl" % prefix[k])
            self._vocabs[k] = pickle.load(open(vfile, "rb"))
            fn = os.path.join(path, "%s.%s" % (prefix[k], file_postfix))
            if not os.path.exists(fn) and os.path.exists(fn + ".gz"):
                fn += ".gz"
            self._lines[k] = read_corpus(fn, skip_empty_lines=False)
            self._unknown[k] = unknown_label.get(k) if isinstance(unknown_label, dict) else unknown_label
            inv = sorted(self._vocabs[k].items(), key=lambda kv: kv[1])
            self.labels[k] = [s for s, _ in inv]
        n = len(self._lines["data"])
        assert all(len(v) == n for v in self._lines.values()), "%s: source and target differ in the number of lines" % self
        self.num_outputs = {k: (max(self._vocabs[k].values()) + 1, 1) for k in self._keys}
        self.num_inputs = self.num_outputs["data"][0]
        self._order: List[int] = []

    def _encode(self, key: str, line: str) -> numpy.ndarray:
        words = line.split()
        if self._add[key]:
            words += self._add[key].split()
        v = self._vocabs[key]
        unk = self._unknown[key]
        ids = []
        for w in words:
            if w in v:
                ids.append(v[w])
            elif unk is not None:
                ids.append(v[unk])
            else:
                raise KeyError("%s: %r not in the %s vocabulary and no unknown_label given" % (self, w, key))
        return numpy.array(ids, dtype="int32")

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        n = len(self._lines["data"])
        if seq_order is not None:
            self._order = list(seq_order)
        elif seq_list is not None:
            self._order = [int(t.split("-")[-1]) for t in seq_list]
        else:
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=n, get_seq_len=lambda i: len(self._lines["data"][i].split())))
        self._num_seqs = len(self._order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._lines["data"])

    def get_all_tags(self):
        return ["line-%i" % i for i in range(len(self._lines["data"]))]

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        line = self._order[seq_idx]
        return DatasetSeq(seq_idx=seq_idx, seq_tag="line-%i" % line, features={k: self._encode(k, self._lines[k][line]) for k in self._keys})

    def get_data_keys(self):
        return list(self._keys)

    def get_target_list(self):
        return [k for k in self._keys if k != "data"]

    def get_data_dtype(self, key):
        return "int32"

    def is_data_sparse(self, key):
        return True

    def get_data_dim(self, key):
        return self.num_outputs[key][0]

    def get_data_shape(self, key):
        return []


class TranslationFactorsDataset(TranslationDataset):
    """
    Parallel text whose words carry extra factors (casing, morphology ...): ``this|u is|l an|l example|u``. Every word of a file has the
    same number of factors. The first source factor is the key ``data``, the first target factor ``classes``; the further ones get the
    keys named in ``source_factors`` / ``target_factors`` and need a vocabulary ``<key>.vocab.pkl`` each.
    Parity: returnn/datasets/lm.py:1895.
    """

    def __init__(self, source_factors: Union[None, str, Sequence[str]] = None, target_factors: Union[None, str, Sequence[str]] = None,
                 factor_separator: str = "|", **kwargs):
        self._source_factors = [source_factors] if isinstance(source_factors, str) else list(source_factors or [])
        self._target_factors = [target_factors] if isinstance(target_factors, str) else list(target_factors or [])
        self._factor_separator = factor_separator
        super().__init__(**kwargs)
        import pickle

        groups = [("data", self._source_factors)] + ([] if self.source_only else [("classes", self._target_factors)])
        self._factor_keys: Dict[str, List[str]] = {}
        for main, extra in groups:
            self._factor_keys[main] = [main] + extra
            for k in extra:
                with open(os.path.join(self.path, "%s.vocab.pkl" % k), "rb") as f:
                    self._vocabs[k] = pickle.load(f)
                self._unknown[k] = self._unknown[main]
                self._add[k] = self._add[main]
                self.labels[k] = [w for w, _ in sorted(self._vocabs[k].items(), key=lambda kv: kv[1])]
                self.num_outputs[k] = (max(self._vocabs[k].values()) + 1, 1)
        self._all_keys = [k for main, _ in groups for k in self._factor_keys[main]]

    def _encode_factors(self, main: str, line: str) -> Dict[str, numpy.ndarray]:
        keys = self._factor_keys[main]
        words = line.split()
        cols: List[List[str]] = [[] for _ in keys]
        for w in words:
            parts = w.split(self._factor_separator)
            assert len(parts) == len(keys), "%s: word %r has %i factors, expected %i (%s)" % (self, w, len(parts), len(keys), ", ".join(keys))
            for c, part in zip(cols, parts):
                c.append(part)
        # the postfix (sentence end etc.) is appended to every factor, as to the main stream
        return {k: self._encode(k, " ".join(c)) for k, c in zip(keys, cols)}

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        line = self._order[seq_idx]
        feats: Dict[str, numpy.ndarray] = {}
        for main in self._factor_keys:
            feats.update(self._encode_factors(main, self._lines[main][line]))
        return DatasetSeq(seq_idx=seq_idx, seq_tag="line-%i" % line, features=feats)

    def get_data_keys(self):
        return list(self._all_keys)

    def get_target_list(self):
        return [k for k in self._all_keys if k not in self._factor_keys["data"]]


class ConfusionNetworkDataset(TranslationDataset):
    """
    Source sentences with weighted alternatives per position (confusion networks):
    ``__ALT__ we're|0.9997__were|0.0003 a|0.98__EPS|0.02 social|1.0 species|1.0``. Positions are separated by blanks, alternatives by two
    underscores, a weight follows each word after ``|``; a line without the ``__ALT__`` mark is plain text (one alternative of weight 1
    per position). Keys: ``sparse_inputs`` (int32 ``[time, max_density]``, unused slots 0), ``sparse_weights`` (float32, unused slots 0)
    and ``classes``. Parity: returnn/datasets/lm.py:2025.
    """

    ALT_MARK = "__ALT__"

    def __init__(self, max_density: int = 20, **kwargs):
        self.density = int(max_density)
        super().__init__(**kwargs)
        self._cn_keys = ["sparse_inputs", "sparse_weights"] + ([] if self.source_only else ["classes"])
        self.num_outputs["sparse_inputs"] = (self.num_outputs["data"][0], 2)
        self.num_outputs["sparse_weights"] = (self.density, 2)
        self.labels["sparse_inputs"] = self.labels["data"]

    def _lookup(self, word: str) -> int:
        v = self._vocabs["data"]
        if word in v:
            return v[word]
        unk = self._unknown["data"]
        if unk is None:
            raise KeyError("%s: %r not in the source vocabulary and no unknown_label given" % (self, word))
        return v[unk]

    def _encode_network(self, line: str):
        words = line.split()
        if words and words[0] == self.ALT_MARK:
            slots = []
            for pos in words[1:]:
                arcs = []
                for arc in pos.split("__"):
                    w, _, weight = arc.rpartition("|")
                    assert w, "%s: alternative %r has no weight" % (self, arc)
                    arcs.append((self._lookup(w), float(weight)))
                slots.append(arcs)
        else:
            slots = [[(self._lookup(w), 1.0)] for w in words]
        for w in self._add["data"].split():
            slots.append([(self._lookup(w), 1.0)])
        ids = numpy.zeros((len(slots), self.density), dtype="int32")
        weights = numpy.zeros((len(slots), self.density), dtype="float32")
        for t, arcs in enumerate(slots):
            assert len(arcs) <= self.density, "%s: %i alternatives at one position, max_density is %i" % (self, len(arcs), self.density)
            for a, (i, wgt) in enumerate(arcs):
                ids[t, a] = i
                weights[t, a] = wgt
        return ids, weights

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        res = super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is None and seq_list is None:
            # lengths for the sorted orders: positions, not alternatives
            n = len(self._lines["data"])
            self._order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=n, get_seq_len=lambda i: len(self._lines["data"][i].split())))
            self._num_seqs = len(self._order)
        return res

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._order):
            return None
        line = self._order[seq_idx]
        ids, weights = self._encode_network(self._lines["data"][line])
        feats = {"sparse_inputs": ids, "sparse_weights": weights}
        if not self.source_only:
            feats["classes"] = self._encode("classes", self._lines["classes"][line])
        return DatasetSeq(seq_idx=seq_idx, seq_tag="line-%i" % line, features=feats)

    def get_data_keys(self):
        return list(self._cn_keys)

    def get_target_list(self):
        return ["classes"] if not self.source_only else []

    def get_data_dtype(self, key):
        return "float32" if key == "sparse_weights" else "int32"

    def is_data_sparse(self, key):
        return key == "classes"

    def get_data_dim(self, key):
        return self.density if key in ("sparse_inputs", "sparse_weights") else self.num_outputs[key][0]

    def get_data_shape(self, key):
        return [self.density] if key in ("sparse_inputs", "sparse_weights") else []


class AllophoneState:
    """
    One HMM state of a context-dependent phone, in RASR's notation ``center{left+right}@i@f.state`` (``@i`` / ``@f``: first / last phone of
    a word). Hashable; :meth:`index` maps it to a dense integer given the phone inventory. Parity: returnn/datasets/lm.py:882.
    """

    def __init__(self, id: Optional[str] = None, state: Optional[int] = None):
        self.id: Optional[str] = id  # centre phone
        self.context_history: Tuple[str, ...] = ()  # left context, nearest phone last
        self.context_future: Tuple[str, ...] = ()  # right context, nearest phone first
        self.boundary = 0  # bit 1: word-initial, bit 2: word-final
        self.state = state
        self._attrs = ("id", "context_history", "context_future", "boundary", "state")

    def format(self) -> str:
        """RASR notation"""
        s = "%s{%s+%s}" % (self.id, "-".join(self.context_history) or "#", "-".join(self.context_future) or "#")
        if self.boundary & 1:
            s += "@i"
        if self.boundary & 2:
            s += "@f"
        if self.state is not None:
            s += ".%i" % self.state
        return s

    __repr__ = format

    def copy(self) -> "AllophoneState":
        """shallow copy"""
        a = AllophoneState(self.id, self.state)
        a.context_history, a.context_future, a.boundary = self.context_history, self.context_future, self.boundary
        return a

    def mark_initial(self):
        """first phone of a word"""
        self.boundary |= 1

    def mark_final(self):
        """last phone of a word"""
        self.boundary |= 2

    def phone_idx(self, ctx_idx: int, phone_idxs: Dict[str, int]) -> int:
        """index of the centre phone (``ctx_idx`` 0) or of a context phone (-1, -2 ... left; 1, 2 ... right), 0 meaning "none", phones from 1"""
        if ctx_idx == 0:
            p = self.id
        elif ctx_idx > 0:
            p = self.context_future[ctx_idx - 1] if ctx_idx - 1 < len(self.context_future) else None
        else:
            p = self.context_history[ctx_idx] if -ctx_idx <= len(self.context_history) else None
        return 0 if p is None else phone_idxs[p] + 1

    def index(self, phone_idxs: Dict[str, int], num_states: int = 3, context_length: int = 1) -> int:
        """
        Dense index over (centre, left and right contexts, boundary, state), mixed radix with the phone inventory + 1 ("none") as the
        base of the phone digits.
        """
        assert self.state is not None and 0 <= self.state < num_states
        base = max(phone_idxs.values()) + 2
        r = 0
        for i in range(2 * context_length + 1):
            ctx = (i + 1) // 2 * (1 if i % 2 else -1)  # 0, 1, -1, 2, -2 ...
            r = r * base + self.phone_idx(ctx, phone_idxs)
        r = r * 4 + self.boundary
        return r * num_states + self.state

    @classmethod
    def from_index(cls, index: int, phone_ids: Dict[int, str], num_states: int = 3, context_length: int = 1) -> "AllophoneState":
        """inverse of :meth:`index` (``phone_ids``: index -> phone)"""
        base = max(phone_ids.keys()) + 2
        a = cls()
        a.state = index % num_states
        index //= num_states
        a.boundary = index % 4
        index //= 4
        digits = []
        for _ in range(2 * context_length + 1):
            digits.append(index % base)
            index //= base
        digits.reverse()
        hist: List[Optional[str]] = [None] * context_length
        fut: List[Optional[str]] = [None] * context_length
        for i, d in enumerate(digits):
            ctx = (i + 1) // 2 * (1 if i % 2 else -1)
            p = phone_ids[d - 1] if d > 0 else None
            if ctx == 0:
                a.id = p
            elif ctx > 0:
                fut[ctx - 1] = p
            else:
                hist[ctx] = p
        a.context_history = tuple(p for p in hist if p is not None)
        a.context_future = tuple(p for p in fut if p is not None)
        return a

    def __hash__(self):
        return hash(tuple(getattr(self, a) for a in self._attrs))

    def __eq__(self, other):
        return isinstance(other, AllophoneState) and all(getattr(self, a) == getattr(other, a) for a in self._attrs)

    def __ne__(self, other):
        return not self == other


class StateTying:
    """
    RASR state-tying file: one ``<allophone state> <class index>`` per line. Parity: returnn/datasets/lm.py:1197.
    """

    def __init__(self, state_tying_file: str):
        self.allo_map: Dict[str, int] = {}  # allophone state notation -> class
        self.class_map: Dict[int, set] = {}  # class -> allophone states
        with _open_text(state_tying_file) as f:
            for line in f:
                line = line.strip()
                if not line or line.startswith("#"):
                    continue
                allo, cls_idx = line.rsplit(None, 1)
                idx = int(cls_idx)
                assert allo not in self.allo_map, "state tying %s: %s listed twice" % (state_tying_file, allo)
                self.allo_map[allo] = idx
                self.class_map.setdefault(idx, set()).add(allo)
        n = max(self.class_map) + 1 if self.class_map else 0
        missing = [i for i in range(n) if i not in self.class_map]
        assert not missing, "state tying %s: classes %r have no allophone state" % (state_tying_file, missing[:10])
        self.num_classes = n


class Lexicon:
    """Bliss lexicon XML: phoneme inventory and ``orth -> [phoneme sequences]``"""

    def __init__(self, filename: str):
        self.filename = filename
        self.phoneme_list: List[str] = []
        self.phonemes: Dict[str, Dict[str, Any]] = {}
        self.lemmas: Dict[str, Dict[str, Any]] = {}
        opener = gzip.open if filename.endswith(".gz") else open
        with opener(filename, "rb") as f:
            root = ElementTree.parse(f).getroot()
        for ph in root.iter("phoneme"):
            sym = ph.findtext("symbol").strip()
            var = (ph.findtext("variation") or "context").strip()
            self.phonemes[sym] = {"index": len(self.phoneme_list), "symbol": sym, "variation": var}
            self.phoneme_list.append(sym)
        for lemma in root.iter("lemma"):
            orths = [(o.text or "").strip() for o in lemma.findall("orth")]
            phons = [{"phon": (p.text or "").strip(), "score": float(p.attrib.get("score", 0.0))} for p in lemma.findall("phon")]
            for orth in orths:
                self.lemmas[orth] = {"orth": orth, "phons": phons}


class PhoneSeqGenerator:
    """random pronunciations of word sequences from a lexicon, with optional silence between words"""

    def __init__(self, lexicon_file: str, allo_num_states: int = 3, allo_context_len: int = 1, state_tying_file: Optional[str] = None,
                 add_silence_beginning: float = 0.1, add_silence_between_words: float = 0.1, add_silence_end: float = 0.1,
                 repetition: float = 0.9, silence_repetition: float = 0.95):
        self.lexicon = Lexicon(lexicon_file)
        self.phonemes = sorted(self.lexicon.phonemes.keys(), key=lambda s: self.lexicon.phonemes[s]["index"])
        self.rnd = numpy.random.RandomState(0)
        self.allo_num_states = allo_num_states
        self.add_silence_beginning, self.add_silence_between_words, self.add_silence_end = add_silence_beginning, add_silence_between_words, add_silence_end
        self.si_phone = "[SILENCE]" if "[SILENCE]" in self.lexicon.phonemes else "si"

    def random_seed(self, seed: int):
        """reseed"""
        self.rnd.seed(seed)

    def generate_seq(self, orth: str) -> List[str]:
        """phoneme symbols for the sentence"""
        out: List[str] = []
        words = orth.split()
        if self.rnd.random_sample() < self.add_silence_beginning:
            out.append(self.si_phone)
        for i, w in enumerate(words):
            lemma = self.lexicon.lemmas[w]
            phon = lemma["phons"][self.rnd.randint(0, len(lemma["phons"]))]["phon"]
            out.extend(phon.split())
            if i < len(words) - 1 and self.rnd.random_sample() < self.add_silence_between_words:
                out.append(self.si_phone)
        if self.rnd.random_sample() < self.add_silence_end:
            out.append(self.si_phone)
        return out

    def seq_to_class_idxs(self, phones: Sequence[str], dtype: str = "int32") -> numpy.ndarray:
        """phoneme indices"""
        return numpy.array([self.lexicon.phonemes[p]["index"] for p in phones], dtype=dtype)


# ---- text post-processing (names as in the reference, returnn/datasets/lm.py:2245-2563) ------------------------------------------

_ABBREVIATIONS = [(re.compile(r"\b%s\." % a, re.IGNORECASE), b) for a, b in [
    ("mrs", "misess"), ("mr", "mister"), ("dr", "doctor"), ("st", "saint"), ("co", "company"), ("jr", "junior"), ("maj", "major"),
    ("gen", "general"), ("drs", "doctors"), ("rev", "reverend"), ("lt", "lieutenant"), ("hon", "honorable"), ("sgt", "sergeant"),
    ("capt", "captain"), ("esq", "esquire"), ("ltd", "limited"), ("col", "colonel"), ("ft", "fort")]]
_WHITESPACE = re.compile(r"\s+")
_SMALL = "zero one two three four five six seven eight nine ten eleven twelve thirteen fourteen fifteen sixteen seventeen eighteen nineteen".split()
_TENS = "zero ten twenty thirty forty fifty sixty seventy eighty ninety".split()


def expand_abbreviations(text: str) -> str:
    """``Mr.`` -> ``mister`` etc."""
    for rx, full in _ABBREVIATIONS:
        text = rx.sub(full, text)
    return text


def lowercase(text: str) -> str:
    """lower case"""
    return text.lower()


def lowercase_keep_special(text: str) -> str:
    """lower case except for ``[...]`` tokens (noise markers and the like)"""
    return re.sub(r"(\[[^\]]*\])|([^\[]+)", lambda m: m.group(1) or m.group(2).lower(), text)


def collapse_whitespace(text: str) -> str:
    """runs of whitespace -> one blank, trimmed"""
    return _WHITESPACE.sub(" ", text).strip()


def convert_to_ascii(text: str) -> str:
    """transliterate to ASCII (``unidecode`` when installed, else drop the accents)"""
    try:
        from unidecode import unidecode

        return unidecode(text)
    except ImportError:
        import unicodedata

        return unicodedata.normalize("NFKD", text).encode("ascii", "ignore").decode("ascii")


def _number_to_words(n: int) -> str:
    if n < 0:
        return "minus " + _number_to_words(-n)
    if n < 20:
        return _SMALL[n]
    if n < 100:
        return _TENS[n // 10] + ("" if n % 10 == 0 else " " + _SMALL[n % 10])
    if n < 1000:
        return _SMALL[n // 100] + " hundred" + ("" if n % 100 == 0 else " " + _number_to_words(n % 100))
    for size, name in ((10 ** 9, "billion"), (10 ** 6, "million"), (1000, "thousand")):
        if n >= size:
            return _number_to_words(n // size) + " " + name + ("" if n % size == 0 else " " + _number_to_words(n % size))
    return str(n)


def normalize_numbers(text: str, with_spacing: bool = False) -> str:
    """digits -> words (integers, ``1,000`` style separators, simple decimals)"""
    text = re.sub(r"(\d),(\d{3})", r"\1\2", text)

    def repl(m):
        whole, frac = m.group(1), m.group(3)
        words = _number_to_words(int(whole))
        if frac:
            words += " point " + " ".join(_SMALL[int(d)] for d in frac)
        return (" %s " % words) if with_spacing else words

    return re.sub(r"(\d+)(\.(\d+))?", repl, text)


def basic_cleaners(text: str) -> str:
    """lower case, whitespace collapsed"""
    return collapse_whitespace(lowercase(text))


def transliteration_cleaners(text: str) -> str:
    """ASCII, lower case, whitespace collapsed"""
    return collapse_whitespace(lowercase(convert_to_ascii(text)))


def english_cleaners(text: str) -> str:
    """ASCII, lower case, numbers and abbreviations written out, whitespace collapsed"""
    return collapse_whitespace(expand_abbreviations(normalize_numbers(lowercase(convert_to_ascii(text)), with_spacing=True)))


def english_cleaners_keep_special(text: str) -> str:
    """as english_cleaners, ``[...]`` tokens untouched"""
    return collapse_whitespace(expand_abbreviations(normalize_numbers(lowercase_keep_special(convert_to_ascii(text)), with_spacing=True)))


def get_remove_chars(chars: str):
    """function that deletes every character of ``chars``"""
    table = {ord(c): None for c in chars}
    return lambda text: text.translate(table)


def get_replace(old: str, new: str):
    """function that replaces ``old`` by ``new``"""
    return lambda text: text.replace(old, new)


def _identity_pp(text: str) -> str:
    return text


def get_post_processor_function(opts):
    """
    Text -> text function from a name of a function of this module (``"english_cleaners"``), an expression that builds one
    (``"get_remove_chars(',/')"``), a callable, or a list of those (applied in order).
    """
    if not opts:
        return _identity_pp
    if callable(opts):
        assert isinstance(opts("test"), str), "%r is not a function str -> str" % (opts,)
        return opts
    if isinstance(opts, str):
        f = eval(opts, globals()) if ("(" in opts or "," in opts) else globals()[opts]
        if isinstance(f, (tuple, list)):
            f = get_post_processor_function(f)
        assert callable(f) and isinstance(f("test"), str), "%r is not a function str -> str" % (opts,)
        return f
    assert isinstance(opts, (tuple, list))
    if len(opts) == 1:
        return get_post_processor_function(opts[0])
    steps = [get_post_processor_function(o) for o in opts]

    def chained(text: str) -> str:
        for step in steps:
            text = step(text)
        return text

    return chained
