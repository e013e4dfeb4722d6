"""
Vocabularies and tokenizers: label list <-> ids, from a vocab file (Python dict literal, pickle, or one label per line),
BPE (apply merges), sampling BPE (BPE dropout), SentencePiece, characters, UTF-8 bytes, HuggingFace tokenizers.

Parity: returnn/datasets/util/vocabulary.py:29-701.
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Union
import os
import sys
import numpy

__all__ = ["Vocabulary", "BytePairEncoding", "SamplingBytePairEncoding", "SentencePieces", "CharacterTargets",
           "Utf8ByteTargets", "HuggingFaceTokenizer"]


class Vocabulary:
    """label <-> id mapping"""

    _cache: Dict[str, Any] = {}

    @classmethod
    def create_vocab(cls, **opts) -> "Vocabulary":
        """by ``class`` name (default Vocabulary), or BPE when ``bpe_file`` is given"""
        opts = dict(opts)
        clz = cls
        if "class" in opts:
            name = opts.pop("class")
            clz = globals()[name] if isinstance(name, str) else name
        elif "bpe_file" in opts:
            clz = BytePairEncoding
        return clz(**opts)

    @classmethod
    def create_vocab_from_labels(cls, labels: Sequence[str], **opts) -> "Vocabulary":
        """from an in-memory label list"""
        return cls(vocab_file=None, labels=list(labels), unknown_label=None, **opts)

    def __init__(self, vocab_file: Optional[str], seq_postfix: Optional[Sequence[int]] = None, unknown_label: Optional[str] = "UNK",
                 bos_label=None, eos_label=None, pad_label=None, control_symbols: Optional[Dict[str, Any]] = None,
                 user_defined_symbols: Optional[Dict[str, Any]] = None, num_labels: Optional[int] = None, labels: Optional[List[str]] = None):
        self.vocab_file = vocab_file
        self.unknown_label = unknown_label
        self.num_labels: Optional[int] = None
        self._vocab: Optional[Dict[str, int]] = None
        self._labels: Optional[List[str]] = None
        if labels is not None:
            self._labels = list(labels)
            self._vocab = {l: i for i, l in enumerate(self._labels)}
            self.num_labels = len(self._labels)
        elif vocab_file:
            self._parse_vocab()
        if num_labels is not None:
            if self.num_labels is None:
                self.num_labels = num_labels
            assert self.num_labels == num_labels, "vocab has %r labels, expected %r" % (self.num_labels, num_labels)
        self.unknown_label_id = self.to_id(unknown_label, allow_none=True) if unknown_label is not None and self._vocab is not None and (
            unknown_label in self._vocab or isinstance(unknown_label, int)) else None
        self.bos_label_id = self.to_id(bos_label, allow_none=True) if bos_label is not None else None
        self.eos_label_id = self.to_id(eos_label, allow_none=True) if eos_label is not None else None
        self.pad_label_id = self.to_id(pad_label, allow_none=True) if pad_label is not None else None
        self.control_symbol_ids = {k: self.to_id(v) for k, v in (control_symbols or {}).items()}
        self.user_defined_symbol_ids = {k: self.to_id(v) for k, v in (user_defined_symbols or {}).items()}
        self.seq_postfix = list(seq_postfix) if seq_postfix else []

    def __repr__(self):
        return "%s(%r, num_labels=%s)" % (self.__class__.__name__, self.vocab_file, self.num_labels)

    def _parse_vocab(self):
        filename = self.vocab_file
        if filename in self._cache:
            self._vocab, self._labels = self._cache[filename]
            self.num_labels = len(self._labels)
            return
        if filename.endswith(".pkl"):
            import pickle

            d = pickle.load(open(filename, "rb"))
        else:
            content = open(filename, "r", encoding="utf8").read()
            if content.lstrip().startswith("{"):
                d = eval(content)
            else:
                labels = content.splitlines()
                d = {l: i for i, l in enumerate(labels)}
        assert isinstance(d, dict), "vocab file %r: expected a dict label -> id" % filename
        labels = {idx: label for label, idx in sorted(d.items())}
        min_label, max_label = min(labels), max(labels)
        assert min_label == 0, "vocab ids must start at 0"
        if len(labels) - 1 != max_label:
            # duplicate ids (e.g. several unknown spellings): keep the first label per id
            labels = {i: labels.get(i, "<unused-%i>" % i) for i in range(max_label + 1)}
        self._vocab = d
        self._labels = [labels[i] for i in range(len(labels))]
        self.num_labels = len(self._labels)
        self._cache[filename] = (self._vocab, self._labels)

    @classmethod
    def create_vocab_dict_from_labels(cls, labels: Sequence[str]) -> Dict[str, int]:
        """label -> id"""
        return {l: i for i, l in enumerate(labels)}

    @property
    def vocab(self) -> Dict[str, int]:
        """label -> id"""
        return self._vocab

    @property
    def labels(self) -> List[str]:
        """id -> label"""
        return self._labels

    def is_id_valid(self, idx: int) -> bool:
        """in range"""
        return 0 <= idx < self.num_labels

    def id_to_label(self, idx: int, default: Optional[str] = None) -> Optional[str]:
        """label of id"""
        if self.is_id_valid(idx):
            return self._labels[idx]
        if default is not None:
            return default
        raise KeyError("id %r out of range" % idx)

    def label_to_id(self, label: str, default=KeyError) -> Optional[int]:
        """id of label"""
        if label in self._vocab:
            return self._vocab[label]
        if default is KeyError:
            raise KeyError("label %r not in vocab" % label)
        return default

    def to_id(self, label, default=KeyError, allow_none: bool = False) -> Optional[int]:
        """label or id -> id"""
        if isinstance(label, str):
            return self.label_to_id(label, default=default)
        if isinstance(label, int):
            if self.is_id_valid(label):
                return label
            if default is KeyError:
                raise KeyError("invalid label id %r" % label)
            return default
        if label is None and allow_none:
            return None
        raise TypeError("invalid label type %r" % type(label))

    def get_seq(self, sentence: str) -> List[int]:
        """whitespace-separated labels -> ids (+ seq_postfix)"""
        segments = sentence.split()
        return self.get_seq_indices(segments) + self.seq_postfix

    def get_seq_indices(self, seq: Sequence[str]) -> List[int]:
        """labels -> ids, unknown mapped to unknown_label"""
        if self.unknown_label is not None and self.unknown_label_id is not None:
            return [self._vocab.get(k, self.unknown_label_id) for k in seq]
        return [self._vocab[k] for k in seq]

    def get_seq_labels(self, seq: Union[Sequence[int], numpy.ndarray]) -> str:
        """ids -> text"""
        labels = self.labels
        if len(labels) < 1000 and all(len(l) == 1 for l in labels):
            return "".join(labels[int(i)] for i in seq)
        return " ".join(labels[int(i)] for i in seq)

    def tf_get_init_variable_func(self, var):
        """not available (torch only)"""
        raise NotImplementedError

    def serialize_labels(self, data: numpy.ndarray) -> str:
        """alias of get_seq_labels"""
        return self.get_seq_labels(data)


class BytePairEncoding(Vocabulary):
    """subword-nmt style BPE: ``bpe_file`` holds the merge operations, ``vocab_file`` the subword vocabulary"""

    def __init__(self, vocab_file: str, bpe_file: str, seq_postfix=None, **kwargs):
        super().__init__(vocab_file=vocab_file, seq_postfix=seq_postfix, **kwargs)
        from ...utils.bpe import StandardBytePairEncoder

        self.bpe = StandardBytePairEncoder(bpe_codes_file=bpe_file, labels=self._labels)

    def get_seq(self, sentence: str) -> List[int]:
        segments = self.bpe.segment_sentence(sentence)
        return self.get_seq_indices(segments) + self.seq_postfix


class SamplingBytePairEncoding(Vocabulary):
    """BPE with random alternative segmentations (BPE dropout style; ``breadth_prob``)"""

    def __init__(self, vocab_file: str, breadth_prob: float, seq_postfix=None, label_postfix_merge_symbol: Optional[str] = None, word_prefix_symbol: Optional[str] = None, **kwargs):
        super().__init__(vocab_file=vocab_file, seq_postfix=seq_postfix, **kwargs)
        from ...utils.bpe import SamplingBytePairEncoder

        self.rnd = numpy.random.RandomState(0)
        self.bpe = SamplingBytePairEncoder(labels=self._labels, breadth_prob=breadth_prob, rnd=self.rnd, unknown_label=self.unknown_label,
                                           label_postfix_merge_symbol=label_postfix_merge_symbol, word_prefix_symbol=word_prefix_symbol)

    def set_random_seed(self, seed: int):
        """reseed"""
        self.rnd.seed(seed)

    def get_seq(self, sentence: str) -> List[int]:
        segments = self.bpe.segment_sentence(sentence)
        return self.get_seq_indices(segments) + self.seq_postfix


class SentencePieces(Vocabulary):
    """SentencePiece model (``model_file``), optional sampling (``enable_sampling``, ``alpha``)"""

    def __init__(self, **opts):
        import sentencepiece as spm

        self._opts = dict(opts)
        self._cache_key = opts.get("model_file")
        control_symbols = opts.pop("control_symbols", None)
        user_defined_symbols = opts.pop("user_defined_symbols", None)
        self.enable_sampling = opts.pop("enable_sampling", False)
        self.alpha = opts.pop("alpha", 0.1)
        self.nbest_size = opts.pop("nbest_size", -1)
        self.add_eos = opts.pop("add_eos", False)
        self.sp = spm.SentencePieceProcessor(model_file=opts["model_file"])
        labels = [self.sp.id_to_piece(i) for i in range(self.sp.vocab_size())]
        super().__init__(vocab_file=None, labels=labels, unknown_label=self.sp.unk_id() if self.sp.unk_id() >= 0 else None,
                         bos_label=self.sp.bos_id() if self.sp.bos_id() >= 0 else None, eos_label=self.sp.eos_id() if self.sp.eos_id() >= 0 else None,
                         pad_label=self.sp.pad_id() if self.sp.pad_id() >= 0 else None, control_symbols=control_symbols,
                         user_defined_symbols=user_defined_symbols)

    def get_seq(self, sentence: str) -> List[int]:
        if self.enable_sampling:
            ids = self.sp.encode(sentence, enable_sampling=True, alpha=self.alpha, nbest_size=self.nbest_size)
        else:
            ids = self.sp.encode(sentence)
        if self.add_eos and self.eos_label_id is not None:
            ids = list(ids) + [self.eos_label_id]
        return list(ids)

    def get_seq_labels(self, seq) -> str:
        return self.sp.decode([int(i) for i in seq])


class CharacterTargets(Vocabulary):
    """characters as labels"""

    def __init__(self, vocab_file: Optional[str], seq_postfix=None, unknown_label="@", labels=None, **kwargs):
        super().__init__(vocab_file=vocab_file, seq_postfix=seq_postfix, unknown_label=unknown_label, labels=labels, **kwargs)

    def get_seq(self, sentence: str) -> List[int]:
        if self.unknown_label is not None and self.unknown_label_id is not None:
            seq = [self._vocab.get(k, self.unknown_label_id) for k in sentence]
        else:
            seq = [self._vocab[k] for k in sentence]
        return seq + self.seq_postfix

    def get_seq_labels(self, seq) -> str:
        return "".join(self._labels[int(i)] for i in seq)


class Utf8ByteTargets(Vocabulary):
    """UTF-8 bytes as labels (256 classes)"""

    def __init__(self, seq_postfix=None):
        super().__init__(vocab_file=None, seq_postfix=seq_postfix, unknown_label=None, labels=[chr(i) for i in range(256)])

    def get_seq(self, sentence: str) -> List[int]:
        return list(sentence.encode("utf8")) + self.seq_postfix

    def get_seq_labels(self, seq) -> str:
        return bytes(int(i) for i in seq).decode("utf8", errors="replace")


class HuggingFaceTokenizer(Vocabulary):
    """tokenizer from the ``transformers`` package (``huggingface_repo_dir``: local dir or hub name)"""

    def __init__(self, *, huggingface_repo_dir: str):
        import transformers

        self._opts = {"huggingface_repo_dir": huggingface_repo_dir}
        self.tokenizer = transformers.AutoTokenizer.from_pretrained(huggingface_repo_dir, trust_remote_code=False)
        vocab = self.tokenizer.get_vocab()
        labels = [None] * (max(vocab.values()) + 1)
        for k, v in vocab.items():
            labels[v] = k
        labels = [l if l is not None else "<unused-%i>" % i for i, l in enumerate(labels)]
        super().__init__(vocab_file=None, labels=labels, unknown_label=self.tokenizer.unk_token_id, bos_label=self.tokenizer.bos_token_id,
                         eos_label=self.tokenizer.eos_token_id, pad_label=self.tokenizer.pad_token_id)

    def get_seq(self, sentence: str) -> List[int]:
        return list(self.tokenizer(sentence)["input_ids"])

    def get_seq_labels(self, seq) -> str:
        return self.tokenizer.decode([int(i) for i in seq])
