"""
Byte-pair-encoding helpers.

* :class:`StandardBytePairEncoder`: applies the merge operations of a subword-nmt codes file (Sennrich et al. 2016) to a
  sentence; rare words end up as several subword units, joined by ``@@`` at the end of every non-final unit.
* :class:`PrefixTree`, :class:`CharSyncSearch`, :class:`DepthFirstSearch`: enumerate (or sample one of) the segmentations of
  a word into labels of a given vocabulary.
* :class:`SamplingBytePairEncoder`: random segmentations for subword regularisation (``breadth_prob`` = probability to
  prefer the shorter unit at every branching point).

Parity: returnn/util/bpe.py (StandardBytePairEncoder :15, BpeOpts :235, PrefixTree :244, CharSyncSearch :299,
DepthFirstSearch :379, SamplingBytePairEncoder :457).
"""

from __future__ import annotations
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple
import re
import numpy

BpePostMergeSymbol = "@@"
BpeEndOfWord = "</w>"


class StandardBytePairEncoder:
    """greedy application of learned merges, lowest merge rank first"""

    _file_cache: Dict[str, Tuple[Tuple[int, ...], Dict[Tuple[str, str], int]]] = {}

    def __init__(self, bpe_codes_file: str, labels: Optional[Sequence[str]] = None):
        """
        :param bpe_codes_file: one merge ``a b`` per line, optional first line ``#version: x.y``
        :param labels: the vocabulary; units outside of it are split further (down to characters)
        """
        self.labels = set(labels) if labels is not None else None
        self._separator = BpePostMergeSymbol
        self._version, self._ranks = self._load(bpe_codes_file)
        self._reverse = {a + b: (a, b) for (a, b) in self._ranks}
        self._cache: Dict[str, Tuple[str, ...]] = {}

    @classmethod
    def _load(cls, filename: str):
        if filename in cls._file_cache:
            return cls._file_cache[filename]
        version: Tuple[int, ...] = (0, 1)
        ranks: Dict[Tuple[str, str], int] = {}
        with open(filename, "r", encoding="utf8") as f:
            for i, line in enumerate(f):
                line = line.rstrip("\r\n")
                if i == 0 and line.startswith("#version:"):
                    version = tuple(int(x) for x in re.sub(r"(\.0+)*$", "", line.split()[-1]).split("."))
                    continue
                parts = line.split()
                if len(parts) != 2:
                    continue
                ranks.setdefault((parts[0], parts[1]), len(ranks))
        cls._file_cache[filename] = (version, ranks)
        return version, ranks

    def _merge_word(self, word: str) -> Tuple[str, ...]:
        """symbols of one word after all applicable merges; the last symbol carries the end-of-word marker internally"""
        if word in self._cache:
            return self._cache[word]
        if self._version == (0, 1):
            syms = list(word) + [BpeEndOfWord]
        else:  # version 0.2: the marker is attached to the last character
            syms = list(word[:-1]) + [word[-1] + BpeEndOfWord]
        while len(syms) > 1:
            best_rank, best_i = None, -1
            for i in range(len(syms) - 1):
                r = self._ranks.get((syms[i], syms[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best_rank, best_i = r, i
            if best_rank is None:
                break
            a, b = syms[best_i], syms[best_i + 1]
            out = []
            i = 0
            while i < len(syms):  # merge every occurrence of the pair
                if i < len(syms) - 1 and syms[i] == a and syms[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(syms[i])
                    i += 1
            syms = out
        # drop the end-of-word marker
        if syms[-1] == BpeEndOfWord:
            syms = syms[:-1]
        elif syms[-1].endswith(BpeEndOfWord):
            syms[-1] = syms[-1][: -len(BpeEndOfWord)]
        if self.labels is not None:
            syms = self._split_to_vocab(syms)
        res = tuple(syms)
        self._cache[word] = res
        return res

    def _split_to_vocab(self, syms: List[str]) -> List[str]:
        """undo merges of units that are not in the vocabulary (with their ``@@`` form for non-final units)"""
        out: List[str] = []
        for pos, s in enumerate(syms):
            final = pos == len(syms) - 1
            out.extend(self._split_rec(s, final))
        return out

    def _split_rec(self, unit: str, final: bool) -> List[str]:
        form = unit if final else unit + self._separator
        if form in self.labels or len(unit) <= 1:
            return [unit]
        key = unit + BpeEndOfWord if final else unit
        pair = self._reverse.get(key) or self._reverse.get(unit)
        if pair is None:
            return [unit]
        left, right = pair
        if right.endswith(BpeEndOfWord):
            right = right[: -len(BpeEndOfWord)]
        if not right:
            return [unit]
        return self._split_rec(left, False) + self._split_rec(right, final)

    def segment_sentence(self, sentence: str) -> List[str]:
        """:return: subword units of the whitespace-separated words, non-final units end with ``@@``"""
        out: List[str] = []
        for word in sentence.split():
            syms = self._merge_word(word)
            out.extend(s + self._separator for s in syms[:-1])
            out.append(syms[-1])
        return out


@dataclass
class BpeOpts:
    """which convention marks word-internal units: a postfix on non-final units (subword-nmt ``@@``) or a prefix on the first unit (SentencePiece ``▁``)"""

    label_postfix_merge_symbol: Optional[str] = None
    word_prefix_symbol: Optional[str] = None


class PrefixTree:
    """trie over the labels; a node is also a tree"""

    def __init__(self, *, prefix: str = "", opts: BpeOpts):
        self.prefix = prefix
        self.arcs: Dict[str, "PrefixTree"] = {}
        self.finished = False  # a label ends here
        self.bpe_finished = False  # a label followed by the merge symbol ends here
        self.opts = opts

    def add(self, postfix: str) -> "PrefixTree":
        """insert a label; :return: its final node"""
        node = self
        merge = self.opts.label_postfix_merge_symbol
        first = True
        rest = postfix
        while True:
            if first and self.opts.word_prefix_symbol and rest.startswith(self.opts.word_prefix_symbol):
                arc = self.opts.word_prefix_symbol
            elif merge and rest == merge:
                arc = merge
            else:
                arc = rest[:1]
            first = False
            rest = rest[len(arc):]
            child = node.arcs.get(arc)
            if child is None:
                child = PrefixTree(prefix=node.prefix + arc, opts=self.opts)
                node.arcs[arc] = child
            if merge and arc == merge and not rest:
                node.bpe_finished = True
            if not rest:
                child.finished = True
                return child
            node = child


def _label_of(node_prefix: str, *, final: bool, opts: BpeOpts) -> str:
    if opts.label_postfix_merge_symbol and not final:
        return node_prefix + opts.label_postfix_merge_symbol
    return node_prefix


def _unit_ok(node: PrefixTree, *, final: bool, opts: BpeOpts) -> bool:
    """can a unit end at this node (as word-final or as word-internal unit)"""
    if opts.label_postfix_merge_symbol:
        return node.finished if final else node.bpe_finished
    return node.finished


class CharSyncSearch:
    """all segmentations of a word, explored character-synchronously"""

    def __init__(self, bpe: PrefixTree, word: str, word_pos: int = 0):
        self.bpe = bpe
        self.opts = bpe.opts
        self.word = (self.opts.word_prefix_symbol or "") + word
        self.word_pos = word_pos

    def search(self) -> List[List[str]]:
        """:return: every sequence of labels that concatenates to the word"""
        word, root, opts = self.word, self.bpe, self.opts
        # hyps: (units so far, current node)
        hyps: List[Tuple[List[str], PrefixTree]] = [([], root)]
        pos = self.word_pos
        n = len(word)
        while pos < n:
            if pos == 0 and opts.word_prefix_symbol and word.startswith(opts.word_prefix_symbol):
                ch = opts.word_prefix_symbol
            else:
                ch = word[pos]
            pos += len(ch)
            nxt: List[Tuple[List[str], PrefixTree]] = []
            for units, node in hyps:
                child = node.arcs.get(ch)
                if child is None:
                    continue
                nxt.append((units, child))
                if pos < n and _unit_ok(child, final=False, opts=opts):
                    nxt.append((units + [_label_of(child.prefix, final=False, opts=opts)], root))
            hyps = nxt
            if not hyps:
                return []
        return [units + [node.prefix] for units, node in hyps if node is not root and _unit_ok(node, final=True, opts=opts)]


class DepthFirstSearch:
    """one segmentation, depth first; at every point where a unit could end, ``sampler()`` decides whether to end it there first"""

    def __init__(self, bpe: PrefixTree, word: str, sampler: Optional[Callable[[], bool]] = None):
        self.bpe = bpe
        self.opts = bpe.opts
        self.word = (self.opts.word_prefix_symbol or "") + word
        self.sampler = sampler

    def search(self) -> Optional[List[str]]:
        """:return: a segmentation or None if the word cannot be written with the labels"""
        word, root, opts = self.word, self.bpe, self.opts
        n = len(word)
        import sys

        if n * 2 + 50 > sys.getrecursionlimit():
            sys.setrecursionlimit(n * 2 + 100)

        def rec(pos: int, node: PrefixTree) -> Optional[List[str]]:
            if pos == n:
                return [node.prefix] if node is not root and _unit_ok(node, final=True, opts=opts) else None
            if pos == 0 and opts.word_prefix_symbol and word.startswith(opts.word_prefix_symbol):
                ch = opts.word_prefix_symbol
            else:
                ch = word[pos]
            child = node.arcs.get(ch)
            if child is None:
                return None
            npos = pos + len(ch)
            options = ["extend"]
            if npos < n and _unit_ok(child, final=False, opts=opts):
                cut_first = bool(self.sampler()) if self.sampler else False
                options = ["cut", "extend"] if cut_first else ["extend", "cut"]
            for opt in options:
                if opt == "extend":
                    r = rec(npos, child)
                    if r is not None:
                        return r
                else:
                    r = rec(npos, root)
                    if r is not None:
                        return [_label_of(child.prefix, final=False, opts=opts)] + r
            return None

        return rec(0, root)


class SamplingBytePairEncoder:
    """random segmentation per word; words without any segmentation map to ``unknown_label``"""

    def __init__(self, *, labels: Sequence[str], breadth_prob: float, rnd: numpy.random.RandomState, unknown_label: Optional[str] = None,
                 opts: Optional[BpeOpts] = None, label_postfix_merge_symbol: Optional[str] = None, word_prefix_symbol: Optional[str] = None):
        """
        :param breadth_prob: 0 = always the longest units (deterministic), 1 = always cut as early as possible
        """
        if opts is None:
            if label_postfix_merge_symbol is None and word_prefix_symbol is None:
                label_postfix_merge_symbol = BpePostMergeSymbol
            opts = BpeOpts(label_postfix_merge_symbol=label_postfix_merge_symbol, word_prefix_symbol=word_prefix_symbol)
        self.opts = opts
        self.labels = list(labels)
        self.unknown_label = unknown_label
        self.breadth_prob = breadth_prob
        self.rnd = rnd
        self._tree = PrefixTree(opts=opts)
        for label in self.labels:
            self._tree.add(label)

    def _sampler(self) -> bool:
        return self.rnd.random_sample() <= self.breadth_prob

    def get_bpe_split_for_word(self, word: str) -> Optional[List[str]]:
        """:return: units or None"""
        return DepthFirstSearch(bpe=self._tree, word=word, sampler=self._sampler).search()

    def segment_sentence(self, sentence: str) -> List[str]:
        """units of all words"""
        out: List[str] = []
        for word in sentence.split():
            units = self.get_bpe_split_for_word(word)
            if units is None:
                assert self.unknown_label is not None, "no segmentation for %r and no unknown_label" % word
                out.append(self.unknown_label)
            else:
                out.extend(units)
        return out
