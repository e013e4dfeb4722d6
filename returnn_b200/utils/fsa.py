"""
Finite-state acceptors on the host: builders for the topologies used in sequence training (CTC, ASG, HMM with
allophone states, n-gram, staircase), and the batch container consumed by the forward-backward and Viterbi kernels
(:mod:`returnn_b200.ops.fsa`).

An edge is ``(from_state, to_state, emission_label, weight)``; weights are negative log scores (0 = free). The batch
container stores all automata of a batch with one shared state numbering: ``edges [4, E]`` = (from, to, emission,
sequence index), ``weights [E]``, ``start_end_states [2, B]``.

Parity: returnn/util/fsa.py (Edge :20, Graph :122, Asg :211, Ctc :325, Hmm :486, Ngram :797, FastBaumWelchBatchFsa :1030,
FastBwFsaShared :1053, get_ctc_fsa_fast_bw :1151, fast_bw_fsa_staircase :1228).
"""

from __future__ import annotations
from typing import Dict, List, Optional, Sequence, Tuple, Union
import itertools
import numpy


class Edge:
    """one transition"""

    __slots__ = ("source_state_idx", "target_state_idx", "label", "weight", "idx_word_in_sentence", "idx_phon_in_word", "idx", "allo_idx", "score")

    def __init__(self, source_state_idx: int, target_state_idx: int, label, weight: float = 0.0):
        self.source_state_idx = source_state_idx
        self.target_state_idx = target_state_idx
        self.label = label
        self.weight = weight
        self.idx_word_in_sentence = None
        self.idx_phon_in_word = None
        self.idx = None
        self.allo_idx = None
        self.score = None

    def as_tuple(self):
        """(from, to, label, weight)"""
        return self.source_state_idx, self.target_state_idx, self.label, self.weight

    def __repr__(self):
        return "Edge(%r, %r, %r, %r)" % self.as_tuple()

    def __eq__(self, other):
        return self.as_tuple() == other.as_tuple()

    def __lt__(self, other):
        return _sort_key(self) < _sort_key(other)

    def __hash__(self):
        return hash(self.as_tuple())


def _sort_key(e: Edge):
    return e.source_state_idx, e.target_state_idx, str(e.label), e.weight


class Graph:
    """the automata built from one sentence ("lemma"): word-level edges plus whatever the builders derive from them"""

    def __init__(self, lemma: Union[str, Sequence[str]]):
        if isinstance(lemma, str):
            self.lemma = lemma.strip()
            self.lem_list = self.lemma.lower().split()
        else:
            self.lem_list = list(lemma)
            self.lemma = " ".join(self.lem_list)
        self.filename = None
        self.num_states = len(self.lem_list) + 1
        self.edges: List[Edge] = [Edge(i, i + 1, w) for i, w in enumerate(self.lem_list)]
        self.num_states_word = self.num_states
        self.edges_word = list(self.edges)
        self.num_states_asg = -1
        self.edges_asg: List[Edge] = []
        self.num_states_ctc = -1
        self.edges_ctc: List[Edge] = []
        self.num_states_hmm = -1
        self.edges_hmm: List[Edge] = []

    def is_empty(self) -> bool:
        """no words"""
        return not self.lem_list

    @staticmethod
    def make_single_state_graph(num_states: int, edges: List[Edge]) -> Tuple[int, List[Edge]]:
        """collapse all states into one (every edge becomes a loop)"""
        return 1, sorted({Edge(0, 0, e.label, e.weight) for e in edges})

    def __repr__(self):
        return "Graph(%r, %i states, %i edges)" % (self.lemma, self.num_states, len(self.edges))


def _label_seq_of_graph(fsa: Graph) -> List[str]:
    """the characters of the sentence (words separated by a space symbol)"""
    return list(" ".join(fsa.lem_list))


class Ctc:
    """CTC topology over the characters of the sentence: optional blank between labels, loops on every state"""

    def __init__(self, fsa: Graph, num_labels: int = 256, label_conversion: bool = False):
        self.fsa = fsa
        self.num_labels = num_labels
        self.label_conversion = label_conversion
        self.blank = "blank"

    def _conv(self, label):
        if not self.label_conversion:
            return label
        return self.num_labels - 1 if label == self.blank else ord(label) % (self.num_labels - 1)

    def run(self):
        """fills ``fsa.edges_ctc`` / ``fsa.num_states_ctc``; states 2i = blank before label i, 2i+1 = label i"""
        labels = _label_seq_of_graph(self.fsa)
        n = len(labels)
        edges: List[Edge] = []
        num_states = 2 * n + 1
        for s in range(num_states):
            is_label = s % 2 == 1
            lab = labels[s // 2] if is_label else self.blank
            edges.append(Edge(s, s, self._conv(lab)))  # loop
            if s + 1 < num_states:
                nxt = labels[(s + 1) // 2] if (s + 1) % 2 == 1 else self.blank
                edges.append(Edge(s, s + 1, self._conv(nxt)))
            if is_label and s + 2 < num_states and labels[s // 2] != labels[s // 2 + 1]:
                edges.append(Edge(s, s + 2, self._conv(labels[s // 2 + 1])))
        # a virtual final state reached from the last label and the last blank
        self.fsa.num_states_ctc = num_states
        self.fsa.edges_ctc = edges
        self.fsa.num_states, self.fsa.edges = num_states, edges
        return self.fsa


class Asg:
    """ASG topology (no blank; repeated characters are written with repetition symbols ``rep1 .. repN``)"""

    def __init__(self, fsa: Graph, num_labels: int = 256, asg_repetition: int = 2, label_conversion: bool = False):
        self.fsa = fsa
        self.num_labels = num_labels
        self.asg_repetition = asg_repetition
        self.label_conversion = label_conversion

    def _conv(self, label):
        if not self.label_conversion:
            return label
        if isinstance(label, str) and label.startswith("rep"):
            return self.num_labels - 1 - self.asg_repetition + int(label[3:])
        return ord(label) % (self.num_labels - self.asg_repetition)

    def run(self):
        """fills ``fsa.edges_asg``: runs of equal characters collapse into the character followed by ``rep<k>``"""
        labels = _label_seq_of_graph(self.fsa)
        seq: List[str] = []
        for ch, grp in itertools.groupby(labels):
            k = len(list(grp))
            while k > 0:
                take = min(k, self.asg_repetition + 1)
                seq.append(ch)
                if take > 1:
                    seq.append("rep%i" % (take - 1))
                k -= take
        edges: List[Edge] = []
        for i, lab in enumerate(seq):
            edges.append(Edge(i, i + 1, self._conv(lab)))
            edges.append(Edge(i + 1, i + 1, self._conv(lab)))  # loop: stay in the label
        self.fsa.num_states_asg = len(seq) + 1
        self.fsa.edges_asg = edges
        self.fsa.num_states, self.fsa.edges = self.fsa.num_states_asg, edges
        return self.fsa


class Hmm:
    """words -> phonemes (lexicon) -> allophone states, each with a loop and a forward transition"""

    def __init__(self, fsa: Graph, depth: int = 6, allo_num_states: int = 3, state_tying_conversion: bool = False):
        self.fsa = fsa
        self.depth = depth
        self.allo_num_states = allo_num_states
        self.state_tying_conversion = state_tying_conversion
        self.lexicon: Optional[Dict[str, List[List[str]]]] = None  # word -> pronunciations (lists of phonemes)
        self.state_tying: Optional[Dict[str, int]] = None  # "phon{left+right}@pos.state" -> class index

    def load_lexicon(self, lexicon: Dict[str, List[List[str]]]):
        """word -> list of pronunciations"""
        self.lexicon = lexicon

    def load_state_tying(self, state_tying: Dict[str, int]):
        """allophone state name -> class"""
        self.state_tying = state_tying

    def run(self):
        """fills ``fsa.edges_hmm``; pronunciation variants become parallel paths between the word boundary states"""
        assert self.lexicon is not None, "load_lexicon first"
        edges: List[Edge] = []
        next_state = len(self.fsa.lem_list) + 1  # word boundary states 0..W keep their numbers

        def emit(phon: str, left: str, right: str, st: int, initial: bool, final: bool):
            name = "%s{%s+%s}%s%s.%i" % (phon, left, right, "@i" if initial else "", "@f" if final else "", st)
            if self.state_tying_conversion:
                assert self.state_tying is not None and name in self.state_tying, "allophone state %r not in the state tying" % name
                return self.state_tying[name]
            return name

        for w, word in enumerate(self.fsa.lem_list):
            prons = self.lexicon.get(word)
            assert prons, "word %r not in the lexicon" % word
            for pron in prons:
                cur = w
                n_units = len(pron) * self.allo_num_states
                unit = 0
                for p, phon in enumerate(pron):
                    left = pron[p - 1] if p > 0 else "#"
                    right = pron[p + 1] if p + 1 < len(pron) else "#"
                    for st in range(self.allo_num_states):
                        unit += 1
                        lab = emit(phon, left, right, st, p == 0, p == len(pron) - 1)
                        tgt = (w + 1) if unit == n_units else next_state
                        if unit != n_units:
                            next_state += 1
                        e = Edge(cur, tgt, lab)
                        e.idx_word_in_sentence, e.idx_phon_in_word, e.allo_idx = w, p, st
                        edges.append(e)
                        edges.append(Edge(tgt, tgt, lab))  # loop
                        cur = tgt
        self.fsa.num_states_hmm = next_state
        self.fsa.edges_hmm = edges
        self.fsa.num_states, self.fsa.edges = next_state, edges
        return self.fsa


class AllPossibleWordsFsa:
    """one state with a loop per lexicon word (all word sequences)"""

    def __init__(self, fsa: Graph):
        self.fsa = fsa
        self.lexicon: Optional[Dict[str, List[List[str]]]] = None

    def run(self):
        """fills ``fsa.edges``"""
        assert self.lexicon is not None
        self.fsa.num_states = 1
        self.fsa.edges = [Edge(0, 0, w) for w in sorted(self.lexicon.keys())]
        self.fsa.lem_list = sorted(self.lexicon.keys())
        return self.fsa


class Ngram:
    """n-gram history automaton over a lemma list: a state per history of n-1 words"""

    def __init__(self, n: int):
        self.n = n
        self.lexicon: Optional[Dict[str, List[List[str]]]] = None
        self.num_states = 0
        self.edges: List[Edge] = []

    def run(self):
        """fills ``edges`` / ``num_states``"""
        assert self.lexicon is not None
        words = sorted(self.lexicon.keys())
        hist_len = self.n - 1
        states: Dict[Tuple[str, ...], int] = {(): 0}
        edges: List[Edge] = []
        frontier = [()]
        while frontier:
            nxt = []
            for h in frontier:
                for w in words:
                    h2 = (h + (w,))[-hist_len:] if hist_len > 0 else ()
                    if h2 not in states:
                        states[h2] = len(states)
                        nxt.append(h2)
                    edges.append(Edge(states[h], states[h2], w))
            frontier = nxt
        self.num_states = len(states)
        self.edges = edges
        return self


def load_lexicon(lexicon_name: str) -> Dict[str, List[List[str]]]:
    """Bliss XML lexicon (optionally gzipped) -> word -> pronunciations"""
    from ..datasets.lm import Lexicon

    lex = Lexicon(lexicon_name)
    return {orth: [p["phon"].split() for p in lemma["phons"]] for orth, lemma in lex.lemmas.items()}


def load_state_tying(state_tying_name: str) -> Dict[str, int]:
    """text file ``<allophone state> <class>`` per line"""
    res = {}
    with open(state_tying_name) as f:
        for line in f:
            parts = line.split()
            if len(parts) == 2:
                res[parts[0]] = int(parts[1])
    return res


class FastBaumWelchBatchFsa:
    """the automata of one batch in the layout of the forward-backward kernels"""

    def __init__(self, edges: numpy.ndarray, weights: numpy.ndarray, start_end_states: numpy.ndarray):
        """
        :param edges: [4, E] int32: from, to, emission, sequence index
        :param weights: [E] float32
        :param start_end_states: [2, B] int32
        """
        assert edges.ndim == 2 and edges.shape[0] == 4
        self.num_edges = edges.shape[1]
        assert weights.shape == (self.num_edges,)
        assert start_end_states.ndim == 2 and start_end_states.shape[0] == 2
        self.num_batch = start_end_states.shape[1]
        self.edges = edges
        self.weights = weights
        self.start_end_states = start_end_states


class FastBwFsaShared:
    """one automaton used for every sequence of the batch"""

    def __init__(self):
        self.num_states = 1
        self.edges: List[Edge] = []

    def add_edge(self, source_state_idx: int, target_state_idx: int, emission_idx: int, weight: float = 0.0):
        """states are created as needed"""
        self.num_states = max(self.num_states, source_state_idx + 1, target_state_idx + 1)
        self.edges.append(Edge(source_state_idx, target_state_idx, emission_idx, weight))

    def add_inf_loop(self, state_idx: int, num_emission_labels: int):
        """a free loop for every emission label"""
        for emission in range(num_emission_labels):
            self.add_edge(state_idx, state_idx, emission)

    def get_num_edges(self, n_batch: int) -> int:
        """in the batch container"""
        return len(self.edges) * n_batch

    def get_edges(self, n_batch: int) -> numpy.ndarray:
        """[4, E * n_batch]; sequence b uses states b * num_states .."""
        e = numpy.array([[x.source_state_idx, x.target_state_idx, x.label] for x in self.edges], dtype="int32").reshape(-1, 3)
        out = numpy.zeros((4, len(self.edges) * n_batch), dtype="int32")
        for b in range(n_batch):
            sl = slice(b * len(self.edges), (b + 1) * len(self.edges))
            out[0, sl] = e[:, 0] + b * self.num_states
            out[1, sl] = e[:, 1] + b * self.num_states
            out[2, sl] = e[:, 2]
            out[3, sl] = b
        return out

    def get_weights(self, n_batch: int) -> numpy.ndarray:
        """[E * n_batch]"""
        return numpy.tile(numpy.array([x.weight for x in self.edges], dtype="float32"), n_batch)

    def get_start_end_states(self, n_batch: int) -> numpy.ndarray:
        """start = state 0, end = last state, per sequence"""
        base = numpy.arange(n_batch, dtype="int32") * self.num_states
        return numpy.stack([base, base + self.num_states - 1])

    def get_fast_bw_fsa(self, n_batch: int) -> FastBaumWelchBatchFsa:
        """the batch container"""
        return FastBaumWelchBatchFsa(self.get_edges(n_batch), self.get_weights(n_batch), self.get_start_end_states(n_batch))


def get_ctc_fsa_fast_bw(*, targets: numpy.ndarray, seq_lens: numpy.ndarray, blank_idx: int, label_loop: bool = True) -> FastBaumWelchBatchFsa:
    """
    CTC automata for a batch of label sequences such that every alignment string has exactly ONE path to the single end
    state.

    :param targets: [B, S]
    :param seq_lens: [B]
    """
    n_batch = targets.shape[0]
    assert seq_lens.shape == (n_batch,)
    edges: List[Tuple[int, int, int, int]] = []
    start_end: List[Tuple[int, int]] = []
    state = 0
    for b in range(n_batch):
        n = int(seq_lens[b])
        labels = [int(x) for x in targets[b, :n]]
        # states: 2i = "before label i, in blank", 2i+1 = "in label i"; final state F entered by the last emission
        base = state
        n_inner = 2 * n + 1
        final = base + n_inner
        for s in range(n_inner):
            is_label = s % 2 == 1
            cur = base + s
            em = labels[s // 2] if is_label else blank_idx
            if not is_label or label_loop:
                edges.append((cur, cur, em, b))
            if s + 1 < n_inner:
                em1 = labels[(s + 1) // 2] if (s + 1) % 2 == 1 else blank_idx
                edges.append((cur, base + s + 1, em1, b))
            if is_label and s + 2 < n_inner and labels[s // 2] != labels[s // 2 + 1]:
                edges.append((cur, base + s + 2, labels[s // 2 + 1], b))
        # one end state: every edge into the last blank or the last label state gets a copy into `final` (no outgoing
        # edges), so a path that ends in one of the two at the last frame corresponds to exactly one path ending in `final`
        ends = {base + n_inner - 1} | ({base + n_inner - 2} if n > 0 else set())
        first_of_seq = next((i for i, e in enumerate(edges) if e[3] == b), len(edges))
        edges.extend([(f, final, em, b) for (f, t, em, _) in edges[first_of_seq:] if t in ends])
        start_end.append((base, final))
        state = final + 1
    e = numpy.array(edges, dtype="int32").T.reshape(4, -1)
    return FastBaumWelchBatchFsa(e, numpy.zeros(e.shape[1], dtype="float32"), numpy.array(start_end, dtype="int32").T.reshape(2, -1))


def fast_bw_fsa_staircase(seq_lens, with_loop: bool = False, max_skip=None, start_max_skip=None, end_max_skip=None) -> FastBaumWelchBatchFsa:
    """
    Staircase automaton per sequence: states 0..n, edge i -> i+1 emits index i; optional loops and skips.

    :param seq_lens: per sequence number of steps n
    :param with_loop: loop on every inner state (emitting the label that led there)
    :param max_skip: allow i -> i+1+k for k <= max_skip (int or per-sequence list); ``start_max_skip`` / ``end_max_skip``: extra
        skips from the start state / into the end state
    """
    n_batch = len(seq_lens)

    def per_batch(v):
        return v if isinstance(v, list) else [v] * n_batch

    max_skip, start_max_skip, end_max_skip = per_batch(max_skip), per_batch(start_max_skip), per_batch(end_max_skip)
    edges: List[Tuple[int, int, int, int]] = []
    start_end = []
    state = 0
    for b in range(n_batch):
        n = int(seq_lens[b])
        base = state
        for i in range(n):
            edges.append((base + i, base + i + 1, i, b))
            if with_loop:
                edges.append((base + i + 1, base + i + 1, i, b))
            skip = max_skip[b] or 0
            if i == 0 and start_max_skip[b] is not None:
                skip = max(skip, start_max_skip[b])
            for k in range(1, skip + 1):
                if i + k < n:
                    edges.append((base + i, base + i + k + 1, i + k, b))
        if end_max_skip[b]:
            for k in range(1, end_max_skip[b] + 1):
                if n - 1 - k >= 0:
                    edges.append((base + n - 1 - k, base + n, n - 1, b))
        start_end.append((base, base + n))
        state = base + n + 1
    e = numpy.array(edges, dtype="int32").T.reshape(4, -1)
    return FastBaumWelchBatchFsa(e, numpy.zeros(e.shape[1], dtype="float32"), numpy.array(start_end, dtype="int32").T.reshape(2, -1))


class Store:
    """
    Writes an automaton to disk: Graphviz source (``.dot``, always) and, when the ``dot`` program is installed, the rendering in
    ``file_format``. Parity: returnn/util/fsa.py:933 (which goes through the ``graphviz`` Python package).
    """

    def __init__(self, num_states: int, edges: Sequence[Edge], filename: str = "edges", path: str = "./tmp/", file_format: str = "svg"):
        self.num_states = num_states
        self.edges = list(edges)
        self.filename = filename
        self.path = path
        self.file_format = file_format
        self.dot_source: Optional[str] = None

    @staticmethod
    def label_conversion(edges: Sequence[Edge]) -> List[Edge]:
        """integer labels back to printable ones where that is unambiguous (characters), everything else as ``str``"""
        out = []
        for e in edges:
            lab = e.label
            if isinstance(lab, (int, numpy.integer)) and 32 <= int(lab) < 127:
                lab = "%s(%i)" % (chr(int(lab)), int(lab))
            out.append(Edge(e.source_state_idx, e.target_state_idx, str(lab), e.weight))
        return out

    def fsa_to_dot_format(self) -> str:
        """Graphviz source: left-to-right, state 0 marked as start, the last state as final"""
        lines = ["digraph fsa {", "  rankdir=LR;", '  node [shape=circle];']
        for s in range(self.num_states):
            shape = "doublecircle" if s == self.num_states - 1 else "circle"
            style = ', style=bold' if s == 0 else ""
            lines.append('  %i [shape=%s%s];' % (s, shape, style))
        for e in self.label_conversion(self.edges):
            label = e.label.replace('"', '\\"')
            if e.weight:
                label += " / %g" % e.weight
            lines.append('  %i -> %i [label="%s"];' % (e.source_state_idx, e.target_state_idx, label))
        lines.append("}")
        self.dot_source = "\n".join(lines) + "\n"
        return self.dot_source

    def save_to_file(self) -> str:
        """
        :return: path of the ``.dot`` file (the rendering, if made, lies beside it with the extension ``file_format``)
        """
        import os
        import shutil
        import subprocess

        if self.dot_source is None:
            self.fsa_to_dot_format()
        os.makedirs(self.path, exist_ok=True)
        dot_path = os.path.join(self.path, self.filename + ".dot")
        with open(dot_path, "w") as f:
            f.write(self.dot_source)
        exe = shutil.which("dot")
        if exe and self.file_format != "dot":
            subprocess.run([exe, "-T" + self.file_format, dot_path, "-o", os.path.join(self.path, "%s.%s" % (self.filename, self.file_format))], check=False)
        return dot_path


def main(argv: Optional[Sequence[str]] = None) -> Graph:
    """
    ``python -m returnn_b200.utils.fsa --fsa {ctc,asg,hmm} --label_seq "hello world" [--file NAME]``: builds the automaton of one
    sentence, prints its size and edges, optionally stores it. Parity: returnn/util/fsa.py:1305.
    """
    import argparse
    import time

    ap = argparse.ArgumentParser(description="automaton of one label sequence")
    ap.add_argument("--fsa", type=str, default="ctc", choices=["ctc", "asg", "hmm"])
    ap.add_argument("--label_seq", type=str, required=True)
    ap.add_argument("--file", type=str)
    ap.add_argument("--path", type=str, default="./tmp/")
    ap.add_argument("--file_format", type=str, default="svg")
    ap.add_argument("--asg_repetition", type=int, default=2)
    ap.add_argument("--num_labels", type=int, default=256)
    ap.add_argument("--label_conversion", dest="label_conversion", action="store_true")
    ap.add_argument("--no_label_conversion", dest="label_conversion", action="store_false")
    ap.set_defaults(label_conversion=False, state_tying_conversion=False, single_state=False, timings=False)
    ap.add_argument("--depth", type=int, default=6)
    ap.add_argument("--allo_num_states", type=int, default=3)
    ap.add_argument("--lexicon", type=str)
    ap.add_argument("--state_tying", type=str)
    ap.add_argument("--state_tying_conversion", dest="state_tying_conversion", action="store_true")
    ap.add_argument("--no_state_tying_conversion", dest="state_tying_conversion", action="store_false")
    ap.add_argument("--single_state", dest="single_state", action="store_true")
    ap.add_argument("--no_single_state", dest="single_state", action="store_false")
    ap.add_argument("--timings", dest="timings", action="store_true")
    ap.add_argument("--ngram", type=int)
    args = ap.parse_args(argv)
    t0 = time.time()
    fsa = Graph(lemma=args.label_seq)
    if args.ngram:
        ngram = Ngram(args.ngram)
        ngram.run()
    if args.fsa == "ctc":
        Ctc(fsa, num_labels=args.num_labels, label_conversion=args.label_conversion).run()
    elif args.fsa == "asg":
        Asg(fsa, num_labels=args.num_labels, asg_repetition=args.asg_repetition, label_conversion=args.label_conversion).run()
    else:
        assert args.lexicon, "--fsa hmm needs --lexicon (and optionally --state_tying)"
        hmm = Hmm(fsa, depth=args.depth, allo_num_states=args.allo_num_states, state_tying_conversion=args.state_tying_conversion)
        hmm.load_lexicon(load_lexicon(args.lexicon))
        if args.state_tying:
            hmm.load_state_tying(load_state_tying(args.state_tying))
        hmm.run()
    num_states, edges = fsa.num_states, fsa.edges
    if args.single_state:
        num_states, edges = Graph.make_single_state_graph(num_states, edges)
    if args.timings:
        print("built in %.3f s" % (time.time() - t0))
    print("%s automaton of %r: %i states, %i edges" % (args.fsa, fsa.lemma, num_states, len(edges)))
    for e in edges:
        print(" ", e.as_tuple())
    if args.file:
        where = Store(num_states, edges, filename=args.file, path=args.path, file_format=args.file_format).save_to_file()
        print("stored:", where)
    return fsa


if __name__ == "__main__":
    main()
