"""
Datasets that generate their data on the fly, deterministically per (epoch seed, sequence index):
synthetic tasks (12AX, episodic copy, XML modeling, variable assignment, number base conversion, copy task),
dummy data (fixed template or from an ``extern_data``-like template), and ``StaticDataset`` over given arrays.

Parity: returnn/datasets/generating.py (GeneratingDataset :22-280, Task12AXDataset :281-371, TaskEpisodicCopy,
TaskXmlModeling, TaskVariableAssignment, TaskNumberBaseConvert, DummyDataset*, DummyGenericDataset :963-1040,
StaticDataset, CopyTaskDataset).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union
import numpy
from .basic import Dataset, DatasetSeq, convert_data_dims
from .cached2 import CachedDataset2
from ..utils.basic import class_idx_seq_to_1_of_k, NumbersDict

__all__ = ["GeneratingDataset", "Task12AXDataset", "TaskEpisodicCopyDataset", "TaskXmlModelingDataset",
           "TaskVariableAssignmentDataset", "TaskNumberBaseConvertDataset", "DummyDataset",
           "DummyDatasetMultipleSequenceLength", "DummyDatasetMultipleDataKeys", "DummyGenericDataset", "StaticDataset",
           "CopyTaskDataset"]


class GeneratingDataset(Dataset):
    """
    Base: subclasses implement ``generate_seq(corpus_seq_idx)`` using ``self.random``, which is reseeded with
    ``(epoch seed, corpus_seq_idx)`` before every call, so any sequence can be regenerated in any process.
    """

    _input_classes: Optional[str] = None
    _output_classes: Optional[str] = None

    def __init__(self, input_dim, output_dim, num_seqs=float("inf"), **kwargs):
        super().__init__(**kwargs)
        assert self.shuffle_frames_of_nseqs == 0
        self._input_dim = input_dim
        self._output_dim = output_dim
        self.num_inputs = input_dim
        out = convert_data_dims(output_dim) if isinstance(output_dim, dict) else {"classes": (output_dim, 1)}
        if "data" not in out and input_dim is not None:
            out["data"] = (input_dim * self.window, 2)
        self.num_outputs = out
        self.expected_load_seq_start = 0
        self._seq_order: Optional[Sequence[int]] = None
        self._num_seqs = num_seqs
        self._total_num_seqs = num_seqs
        self.random = numpy.random.RandomState(1)
        self.reached_final_seq = False
        self.added_data: List[DatasetSeq] = []
        if self.seq_ordering in ("sorted", "sorted_reverse"):
            # lengths are not known without generating everything: fall back silently (eval sets ask for sorted)
            self.seq_ordering = "default"

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch)
        self.random.seed(self._get_random_seed_for_epoch(epoch=epoch))
        if seq_list is not None:
            assert seq_order is None
            seq_order = []
            for tag in seq_list:
                assert tag.startswith("seq-") and tag[len("seq-"):].isdigit()
                seq_order.append(int(tag[len("seq-"):]))
        if seq_order is not None:
            self._seq_order = seq_order
            self._num_seqs = len(seq_order)
        elif self._total_num_seqs == float("inf"):
            assert self.seq_ordering == "default"
            self._seq_order = None
            self._num_seqs = self._total_num_seqs
        else:
            self._seq_order = self.get_seq_order_for_epoch(epoch=epoch, num_seqs=self._total_num_seqs, get_seq_len=None)
            self._num_seqs = len(self._seq_order)
        self._num_timesteps = 0
        self.reached_final_seq = False
        self.expected_load_seq_start = 0
        self.added_data = []
        return True

    def supports_sharding(self) -> bool:
        return True

    def _get_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        for data in self.added_data:
            if data.seq_idx == seq_idx:
                return data
        return None

    def is_cached(self, start, end):
        return False

    def _load_seqs(self, start: int, end: int):
        assert start >= self.expected_load_seq_start
        if start > self.expected_load_seq_start:
            i = 0
            while i < len(self.added_data) and self.added_data[i].seq_idx < start:
                i += 1
            del self.added_data[:i]
            self.expected_load_seq_start = start
        if self.added_data:
            start = max(self.added_data[-1].seq_idx + 1, start)
        if end > self.num_seqs:
            end = self.num_seqs
        if end >= self.num_seqs:
            self.reached_final_seq = True
        seqs = [self._make_seq(i) for i in range(start, int(end))]
        for s in seqs:
            nf = s.num_frames
            self._num_timesteps += nf.get("data", nf.max_value() if nf.has_values() else 0)
        self.added_data += seqs

    def _make_seq(self, seq_idx: int) -> DatasetSeq:
        seq = self.get_corpus_seq(self.get_corpus_seq_idx(seq_idx))
        seq.seq_idx = seq_idx
        return seq

    def have_get_corpus_seq(self) -> bool:
        return True

    def get_corpus_seq(self, corpus_seq_idx: int) -> DatasetSeq:
        """deterministic in (epoch seed, corpus_seq_idx)"""
        self.random.seed((self._get_random_seed_for_epoch(epoch=self.epoch), corpus_seq_idx))
        seq = self.generate_seq(corpus_seq_idx)
        if self.window > 1:
            seq.features["data"] = self._sliding_window(seq.features["data"])
        return seq

    def _sliding_window(self, x: numpy.ndarray) -> numpy.ndarray:
        w = int(self.window)
        half = w // 2
        padded = numpy.concatenate([numpy.zeros((half,) + x.shape[1:], x.dtype), x, numpy.zeros((w - 1 - half,) + x.shape[1:], x.dtype)], axis=0)
        return numpy.concatenate([padded[i: i + x.shape[0]] for i in range(w)], axis=1)

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        """:param seq_idx: corpus seq idx"""
        raise NotImplementedError

    def get_num_timesteps(self):
        assert self.reached_final_seq
        return self._num_timesteps

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return self._total_num_seqs

    def have_corpus_seq_idx(self):
        return True

    def get_corpus_seq_idx(self, seq_idx: int) -> int:
        if self._seq_order is None:
            return seq_idx
        return int(self._seq_order[seq_idx])

    def get_seq_length(self, seq_idx):
        assert seq_idx >= self.expected_load_seq_start
        self.load_seqs(self.expected_load_seq_start, seq_idx + 1)
        return self._get_seq(seq_idx).num_frames

    def get_data(self, seq_idx, key):
        return self._get_seq(seq_idx).features[key]

    def get_tag(self, seq_idx):
        seq = self._get_seq(seq_idx)
        if seq is None:
            raise Exception("seq_idx %i not loaded" % seq_idx)
        return seq.seq_tag

    def get_all_tags(self):
        return ["seq-%i" % i for i in range(self.get_total_num_seqs())]

    def get_current_seq_order(self) -> Sequence[int]:
        return self._seq_order

    def get_target_list(self):
        return [k for k in self.num_outputs if k != "data"]

    def get_data_keys(self):
        return (["data"] if "data" in self.num_outputs else []) + self.get_target_list()


class Task12AXDataset(GeneratingDataset):
    """
    12AX working-memory task (O'Reilly & Frank 2006). Input symbols ``1 2 3 A B C X Y Z`` (one-hot, dim 9).
    The target is R at an X that closes ``A..X`` while the last digit was 1, or at a Y that closes ``B..Y`` while the
    last digit was 2; L everywhere else. Sequence lengths are uniform in [10, 100).
    """

    _input_classes = "123ABCXYZ"
    _output_classes = "LR"

    def __init__(self, **kwargs):
        super().__init__(input_dim=len(self._input_classes), output_dim=len(self._output_classes), **kwargs)
        self.labels = {"classes": list(self._output_classes)}

    def get_random_seq_len(self) -> int:
        """uniform 10..99"""
        return self.random.randint(10, 100)

    def generate_input_seq(self, seq_len: int) -> List[int]:
        """symbol distribution biased so that R targets are not too rare"""
        rnd = self.random
        seq = rnd.choice(["", "1", "2"])
        while len(seq) < seq_len:
            if rnd.uniform() < 0.5:
                seq += rnd.choice(list("12"))
            if rnd.uniform() < 0.9:
                seq += rnd.choice(["AX", "BY"])
            while rnd.uniform() < 0.5:
                seq += rnd.choice(list(self._input_classes))
        return [self._input_classes.index(c) for c in seq[:seq_len]]

    @classmethod
    def make_output_seq(cls, input_seq: Sequence[int]) -> List[int]:
        """the 12AX rule"""
        digit, letter = "", ""
        out = []
        for i in input_seq:
            c = cls._input_classes[i]
            hit = False
            if c in "12":
                digit = c
            elif c in "AB":
                letter = c
            elif c in "XY":
                hit = (digit + letter + c) in ("1AX", "2BY")
                letter = ""
            out.append(1 if hit else 0)
        return out

    def estimate_output_class_priors(self, num_trials: int, seq_len: int = 10) -> Tuple[float, float]:
        """empirical (p(L), p(R))"""
        n_r = 0
        for _ in range(num_trials):
            n_r += sum(self.make_output_seq(self.generate_input_seq(seq_len)))
        total = float(num_trials * seq_len)
        return (total - n_r) / total, n_r / total

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        seq_len = self.get_random_seq_len()
        input_seq = self.generate_input_seq(seq_len)
        features = class_idx_seq_to_1_of_k(input_seq, num_classes=len(self._input_classes))
        targets = numpy.array(self.make_output_seq(input_seq), dtype="int32")
        return DatasetSeq(seq_idx=seq_idx, features=features, targets=targets)


class _CharTaskDataset(GeneratingDataset):
    """
    Character-level memory tasks: the input is a string over ``_input_classes`` (one-hot), the target a string of the same length
    over the same alphabet, computed from the input by a small state machine (``make_output_seq``). The alphabets, the order of
    the random draws and the target rules follow the reference exactly, so that a seed gives the same data in both frameworks
    (returnn/datasets/generating.py:374-674).
    """

    _input_classes = ""
    _output_classes = ""

    def __init__(self, **kwargs):
        super().__init__(input_dim=len(self._input_classes), output_dim=len(self._output_classes), **kwargs)
        self.labels = {"classes": list(self._output_classes)}

    def _draw_word(self, alphabet: str, length: int) -> str:
        """``length`` characters, one ``choice`` draw each"""
        letters = list(alphabet)
        return "".join(self.random.choice(letters) for _ in range(length))

    def generate_input_seq(self) -> List[int]:
        """class indices of a random input string"""
        raise NotImplementedError

    @classmethod
    def make_output_seq(cls, input_seq: Sequence[int]) -> List[int]:
        """class indices of the target string for an input"""
        raise NotImplementedError

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        input_seq = self.generate_input_seq()
        features = class_idx_seq_to_1_of_k(input_seq, num_classes=len(self._input_classes))
        return DatasetSeq(seq_idx=seq_idx, features=features, targets=numpy.array(self.make_output_seq(input_seq)))


class TaskEpisodicCopyDataset(_CharTaskDataset):
    """
    Episodic copy (Arjovsky et al. 2015, https://arxiv.org/abs/1511.06464) with random lengths: 1-9 digits to remember, 1-99
    blanks, a delimiter ``.``, then one ``.`` per digit plus one. Target: blank while reading; from the delimiter on the
    remembered digits one by one, then ``.``.
    """

    _input_classes = " .01234567"
    _output_classes = _input_classes

    def generate_input_seq(self) -> List[int]:
        n_chars = self.random.randint(1, 10)
        text = self._draw_word(self._input_classes[2:], n_chars)
        text += " " * self.random.randint(1, 100)
        text += "." + "." * (n_chars + 1)
        return [self._input_classes.index(c) for c in text]

    @classmethod
    def make_output_seq(cls, input_seq: Sequence[int]) -> List[int]:
        memory: List[str] = []
        recalling = False
        out = []
        for idx in input_seq:
            c = cls._input_classes[idx]
            if not recalling:
                out.append(" ")
                if c == ".":
                    recalling = True
                elif c != " ":
                    memory.append(c)
            else:
                out.append(memory.pop(0) if memory else ".")
        return [cls._output_classes.index(c) for c in out]


class TaskXmlModelingDataset(_CharTaskDataset):
    """
    XML modelling (Jozefowicz et al. 2015): nested tags with names of 1-9 letters, at most ``limit_stack_depth`` open at once.
    Target: ``<`` where a tag must start, the letters of the closing tag's name (known from the stack) and its ``>``; blank where the
    next character cannot be known (inside opening tags).
    """

    _input_classes = " <>/abcdefgh"
    _output_classes = _input_classes

    def __init__(self, limit_stack_depth: int = 4, **kwargs):
        super().__init__(**kwargs)
        self.limit_stack_depth = limit_stack_depth

    def generate_input_seq(self) -> List[int]:
        text = " "  # a prediction task: the target at the leading blank is the first character
        open_tags: List[str] = []
        while True:
            if not open_tags or (len(open_tags) < self.limit_stack_depth and self.random.rand() > 0.6):
                name = self._draw_word(self._input_classes[4:], self.random.randint(1, 10))
                text += "<%s>" % name
                open_tags.append(name)
            else:
                text += "</%s>" % open_tags.pop()
            if not open_tags and self.random.rand() > 0.2:
                break
        return [self._input_classes.index(c) for c in text]

    @classmethod
    def make_output_seq(cls, input_seq: Sequence[int]) -> List[int]:
        text = "".join(cls._input_classes[i] for i in input_seq)
        EXPECT_LT, AFTER_LT, IN_OPEN, IN_CLOSE = "expect<", "after<", "open", "close"
        state = None
        stack: List[str] = []  # per open tag: what of its name is still to be emitted when it closes
        out = []
        for c in text:
            if c in " >" and state != IN_CLOSE:
                assert state != EXPECT_LT, repr(text)
                out.append("<")
                state = EXPECT_LT
            elif state == EXPECT_LT:
                assert c == "<", repr(text)
                out.append(" ")
                state = AFTER_LT
            elif state == AFTER_LT:
                if c == "/":
                    assert stack, repr(text)
                    out.append(stack[-1][0])
                    stack[-1] = stack[-1][1:]
                    state = IN_CLOSE
                else:
                    assert c not in " <>/", repr(text)
                    out.append(" ")
                    stack.append(c)
                    state = IN_OPEN
            elif state == IN_OPEN:
                out.append(" ")
                stack[-1] += c
            elif state == IN_CLOSE:
                assert stack, repr(text)
                if stack[-1]:
                    out.append(stack[-1][0])
                    stack[-1] = stack[-1][1:]
                else:
                    out.append(">")
                    stack.pop()
                    state = None
            else:
                raise AssertionError("unexpected %r in %r" % (c, text))
        return [cls._output_classes.index(c) for c in out]


class TaskVariableAssignmentDataset(_CharTaskDataset):
    """
    Variable assignment (key-value retrieval, from the Associative LSTM paper): 1-4 stores ``S(key,value)`` with unique keys of
    2-4 letters and values of 1 letter, then one query ``Q(key)`` followed by the value and ``.``. Target: blank everywhere except
    after the query's ``)``, where the value is spelled out, then ``.``.
    """

    _input_classes = " ,.SQ()abcdefgh"
    _output_classes = _input_classes

    def generate_input_seq(self) -> List[int]:
        letters = self._input_classes[7:]
        store: Dict[str, str] = {}
        parts = []
        for _ in range(self.random.randint(1, 5)):
            key_len = self.random.randint(2, 5)
            while True:
                key = self._draw_word(letters, key_len)
                if key not in store:
                    break
            value = self._draw_word(letters, self.random.randint(1, 2))
            parts.append("S(%s,%s)" % (key, value))
            store[key] = value
        key = self.random.choice(list(store.keys()))
        text = ",".join(parts) + ",Q(%s)%s." % (key, store[key])
        return [self._input_classes.index(c) for c in text]

    @classmethod
    def make_output_seq(cls, input_seq: Sequence[int]) -> List[int]:
        text = "".join(cls._input_classes[i] for i in input_seq)
        store: Dict[str, str] = {}
        out = []
        mode, key, value = "idle", "", ""
        for c in text:
            emit = " "
            if mode == "idle":
                key = ""
                if c == "S":
                    mode = "store("
                elif c == "Q":
                    mode = "query("
                else:
                    assert c in " ,", repr(text)
            elif mode in ("store(", "query("):
                assert c == "(", repr(text)
                mode = "store-key" if mode == "store(" else "query-key"
            elif mode == "store-key":
                if c == ",":
                    assert key
                    value, mode = "", "store-value"
                else:
                    key += c
            elif mode == "store-value":
                if c == ")":
                    assert value
                    store[key] = value
                    mode = "idle"
                else:
                    value += c
            elif mode == "query-key":
                if c == ")":
                    value = store[key]
                    emit, value, mode = value[0], value[1:], "answer"
                else:
                    key += c
            elif mode == "answer":
                if value:
                    emit, value = value[0], value[1:]
                else:
                    emit, mode = ".", "end"
            elif mode == "end":
                assert c == ".", repr(text)
            out.append(emit)
        return [cls._output_classes.index(c) for c in out]


class TaskNumberBaseConvertDataset(GeneratingDataset):
    """
    Convert a number written in ``input_base`` digits into ``output_base`` digits (sequence to sequence, different lengths).
    Reference: returnn/datasets/generating.py:677-745.
    """

    def __init__(self, input_base: int = 8, output_base: int = 2, min_input_seq_len: int = 1, max_input_seq_len: int = 8, **kwargs):
        super().__init__(input_dim=input_base, output_dim={"data": (input_base, 1), "classes": (output_base, 1)}, **kwargs)
        chars = "0123456789abcdefghijklmnopqrstuvwxyz"
        assert 2 <= input_base <= len(chars) and 2 <= output_base <= len(chars)
        assert 0 < min_input_seq_len <= max_input_seq_len
        self.input_base, self.output_base = input_base, output_base
        self._input_classes = chars[:input_base]
        self._output_classes = chars[:output_base]
        self.labels = {"data": self._input_classes, "classes": self._output_classes}
        self.min_input_seq_len, self.max_input_seq_len = min_input_seq_len, max_input_seq_len

    def get_random_input_seq_len(self) -> int:
        """uniform in [min, max]"""
        return self.random.randint(self.min_input_seq_len, self.max_input_seq_len + 1)

    def generate_input_seq(self) -> List[int]:
        """digits, most significant first"""
        return [self.random.randint(0, len(self._input_classes)) for _ in range(self.get_random_input_seq_len())]

    def make_output_seq(self, input_seq: Sequence[int]) -> List[int]:
        """the same number in the output base (``[0]`` for zero)"""
        value = 0
        for d in input_seq:
            value = value * self.input_base + int(d)
        out: List[int] = []
        while value:
            out.insert(0, value % self.output_base)
            value //= self.output_base
        return out or [0]

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        input_seq = self.generate_input_seq()
        return DatasetSeq(seq_idx=seq_idx, features=numpy.array(input_seq), targets=numpy.array(self.make_output_seq(input_seq)))


class DummyDataset(GeneratingDataset):
    """random class sequence; the features are a fixed random embedding of the class plus nothing else (learnable)"""

    def __init__(self, input_dim: int, output_dim: int, num_seqs, seq_len: int = 2, input_max_value: float = 10.0,
                 input_shift=None, input_scale=None, **kwargs):
        super().__init__(input_dim=input_dim, output_dim=output_dim, num_seqs=num_seqs, **kwargs)
        self.seq_len = seq_len
        self.input_max_value = input_max_value
        if input_shift is None:
            input_shift = -input_max_value / 2.0
        self.input_shift = input_shift
        if input_scale is None:
            input_scale = 1.0 / self.input_max_value
        self.input_scale = input_scale

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        seq_len = self.seq_len
        i1 = seq_idx
        i2 = i1 + seq_len * self.num_inputs
        features = numpy.array([((i % self.input_max_value) + self.input_shift) * self.input_scale for i in range(i1, i2)], dtype="float32").reshape((seq_len, self.num_inputs))
        n_out = self.num_outputs["classes"][0]
        i1, i2 = i2, i2 + seq_len
        targets = numpy.array([i % n_out for i in range(i1, i2)], dtype="int32")
        return DatasetSeq(seq_idx=seq_idx, features=features, targets=targets)


class DummyDatasetMultipleSequenceLength(DummyDataset):
    """like DummyDataset with a different length per data key (e.g. encoder-decoder dummy)"""

    def __init__(self, input_dim, output_dim, num_seqs, seq_len=None, input_max_value=10.0, input_shift=None, input_scale=None, **kwargs):
        if seq_len is None:
            seq_len = {"data": 10, "classes": 20}
        super().__init__(input_dim=input_dim, output_dim=output_dim, num_seqs=num_seqs, seq_len=seq_len,
                         input_max_value=input_max_value, input_shift=input_shift, input_scale=input_scale, **kwargs)

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        assert isinstance(self.seq_len, dict)
        n_in, n_cls = self.seq_len["data"], self.seq_len["classes"]
        i1 = seq_idx
        i2 = i1 + n_in * self.num_inputs
        features = numpy.array([((i % self.input_max_value) + self.input_shift) * self.input_scale for i in range(i1, i2)], dtype="float32").reshape((n_in, self.num_inputs))
        n_out = self.num_outputs["classes"][0]
        targets = numpy.array([i % n_out for i in range(i2, i2 + n_cls)], dtype="int32")
        return DatasetSeq(seq_idx=seq_idx, features=features, targets=targets)


class DummyDatasetMultipleDataKeys(DummyDataset):
    """several input and output keys with individual lengths"""

    def __init__(self, output_dim, num_seqs, seq_len=None, input_max_value=10.0, input_shift=None, input_scale=None, data_keys=None, **kwargs):
        if data_keys is None:
            data_keys = ["data", "classes"]
        self.data_keys = data_keys
        if seq_len is None:
            seq_len = {k: 10 for k in data_keys}
        super().__init__(input_dim=None, output_dim=output_dim, num_seqs=num_seqs, seq_len=seq_len,
                         input_max_value=input_max_value, input_shift=input_shift, input_scale=input_scale, **kwargs)

    def get_data_keys(self):
        return list(self.data_keys)

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        features = {}
        i1 = seq_idx
        for key in self.data_keys:
            n = self.seq_len[key]
            dim, ndim = self.num_outputs[key]
            if ndim >= 2:
                i2 = i1 + n * dim
                features[key] = numpy.array([((i % self.input_max_value) + self.input_shift) * self.input_scale for i in range(i1, i2)], dtype="float32").reshape((n, dim))
            else:
                i2 = i1 + n
                features[key] = numpy.array([i % dim for i in range(i1, i2)], dtype="int32")
            i1 = i2
        return DatasetSeq(seq_idx=seq_idx, features=features)


class DummyGenericDataset(GeneratingDataset):
    """
    Random data for an ``extern_data``-like template: normal floats, uniform class indices; the length of every dynamic
    dim is fixed or uniform in ``[lo, hi]``, consistent across the keys that share the dim.
    ``seq_lens``: int | (lo, hi) | {key-or-Dim-or-None: int | (lo, hi)}; a 3-tuple value ``(ref_key, lo_frac, hi_frac)``
    makes a dim's length a random fraction of the length of another key's first dynamic dim.
    """

    def __init__(self, data_template, num_seqs: int, *, seq_lens=None, **kwargs):
        from ..tensor import TensorDict

        tmpl = TensorDict()
        tmpl.update(data_template, auto_convert=True)
        old_style = {k: (v.dim, v.batch_ndim - (1 if v.have_batch_axis() else 0) + (0 if v.sparse else 0)) for k, v in tmpl.data.items()}
        old_style = {k: (v.dim, len([d for d in v.dims if not d.is_batch_dim()])) for k, v in tmpl.data.items()}
        super().__init__(input_dim=None, output_dim=old_style, num_seqs=num_seqs, **kwargs)
        self.data_template = tmpl
        self.seq_lens = seq_lens

    def get_data_keys(self) -> List[str]:
        return list(self.data_template.data.keys())

    def get_target_list(self) -> List[str]:
        res = []
        if "classes" in self.data_template.data:
            res.append("classes")
        res.extend(k for k, v in self.data_template.data.items() if not v.available_for_inference and k != "classes")
        return res

    def get_data_dtype(self, key: str) -> str:
        return self.data_template.data[key].dtype

    def is_data_sparse(self, key: str) -> bool:
        return self.data_template.data[key].sparse

    def get_data_dim(self, key: str) -> int:
        return self.data_template.data[key].dim or 0

    def get_data_shape(self, key: str) -> List[int]:
        return list(self.data_template.data[key].shape[1:])

    def get_extern_data(self):
        return {k: v.get_kwargs() for k, v in self.data_template.data.items()}

    def _len_spec(self, key: str, dim):
        sl = self.seq_lens
        if isinstance(sl, dict):
            for cand in (dim, key, getattr(dim, "name", None), None):
                if cand in sl:
                    return sl[cand]
            return (5, 15)
        if sl is None:
            return (5, 15)
        return sl

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        rnd = self.random
        lens: Dict[Any, int] = {}
        first_dyn_len: Dict[str, int] = {}
        deferred = []
        for key, templ in self.data_template.data.items():
            for dim in templ.dims:
                if dim.is_batch_dim() or dim.is_static() or dim in lens:
                    continue
                spec = self._len_spec(key, dim)
                if isinstance(spec, (tuple, list)) and len(spec) == 3 and isinstance(spec[0], str):
                    deferred.append((key, dim, spec))
                    continue
                lens[dim] = int(spec) if isinstance(spec, int) else int(rnd.randint(spec[0], spec[1] + 1))
                first_dyn_len.setdefault(key, lens[dim])
        for key, dim, (ref, lo, hi) in deferred:
            base = first_dyn_len[ref]
            lens[dim] = max(1, int(round(base * rnd.uniform(lo, hi))))
        feats = {}
        for key, templ in self.data_template.data.items():
            shape = [lens[d] if d.is_dynamic() else d.dimension for d in templ.dims if not d.is_batch_dim()]
            if templ.sparse_dim:
                feats[key] = rnd.randint(0, templ.sparse_dim.dimension, shape).astype(templ.dtype)
            elif templ.dtype.startswith("float"):
                feats[key] = rnd.standard_normal(shape).astype(templ.dtype)
            elif templ.dtype.startswith("int") or templ.dtype.startswith("uint"):
                feats[key] = rnd.randint(0, 10, shape).astype(templ.dtype)
            else:
                raise NotImplementedError("%s generate: data key %r template %s" % (self, key, templ))
        return DatasetSeq(seq_idx=seq_idx, features=feats)


class StaticDataset(CachedDataset2):
    """all data given as a list of dicts of numpy arrays"""

    @classmethod
    def copy_from_dataset(cls, dataset: Dataset, start_seq_idx: int = 0, max_seqs: Optional[int] = None) -> "StaticDataset":
        """materialise (part of) another dataset"""
        if isinstance(dataset, StaticDataset):
            return cls(data=dataset.data, target_list=dataset.target_list, output_dim=dataset.num_outputs, input_dim=dataset.num_inputs)
        seq_idx = start_seq_idx
        data = []
        while dataset.is_less_than_num_seqs(seq_idx):
            dataset.load_seqs(seq_idx, seq_idx + 1)
            if max_seqs is not None and len(data) >= max_seqs:
                break
            data.append({k: dataset.get_data(seq_idx, k) for k in dataset.get_data_keys()})
            seq_idx += 1
        return cls(data=data, target_list=dataset.get_target_list(), output_dim=dataset.num_outputs, input_dim=dataset.num_inputs)

    def __init__(self, data: List[Dict[str, numpy.ndarray]], target_list=None, input_dim=None, output_dim=None, **kwargs):
        super().__init__(**kwargs)
        assert len(data) > 0
        self.data = data
        first = data[0]
        self.data_keys = sorted(first.keys())
        if "data" in self.data_keys:
            self.data_keys.remove("data")
            self.data_keys.insert(0, "data")
        if target_list is None:
            target_list = [k for k in self.data_keys if k not in ("data", "seq_tag")]
        self.target_list = target_list
        if output_dim is None:
            output_dim = {}
        output_dim = convert_data_dims(output_dim)
        if input_dim is not None and "data" not in output_dim:
            output_dim["data"] = (input_dim, 2)
        for key, value in first.items():
            if key == "seq_tag":
                continue
            arr = numpy.asarray(value)
            if key not in output_dim:
                output_dim[key] = (arr.shape[-1] if arr.ndim >= 2 else 0, arr.ndim)
        self.num_inputs = output_dim["data"][0] if "data" in output_dim else 0
        self.num_outputs = output_dim
        self._seq_order = None
        self._total = len(data)

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._seq_order = list(seq_order)
        elif seq_list is not None:
            tags = self.get_all_tags()
            idx = {t: i for i, t in enumerate(tags)}
            self._seq_order = [idx[t] for t in seq_list]
        elif epoch is None:
            self._seq_order = []
        else:
            self._seq_order = list(self.get_seq_order_for_epoch(epoch=epoch, num_seqs=len(self.data),
                                                                get_seq_len=lambda i: len(self.data[i][self.data_keys[0]])))
        self._num_seqs = len(self._seq_order)
        return True

    def supports_seq_order_sorting(self) -> bool:
        return True

    def supports_sharding(self) -> bool:
        return True

    def _collect_single_seq(self, seq_idx):
        if seq_idx >= len(self._seq_order):
            return None
        ci = self._seq_order[seq_idx]
        d = self.data[ci]
        feats = {k: numpy.asarray(v) for k, v in d.items() if k != "seq_tag"}
        return DatasetSeq(seq_idx=seq_idx, features=feats, seq_tag=d.get("seq_tag", "seq-%i" % ci))

    @property
    def num_seqs(self):
        return self._num_seqs

    def get_total_num_seqs(self, *, fast=False):
        return len(self.data)

    def get_all_tags(self):
        return [d.get("seq_tag", "seq-%i" % i) for i, d in enumerate(self.data)]

    def get_data_keys(self):
        return [k for k in self.data_keys if k != "seq_tag"]

    def get_target_list(self):
        return self.target_list

    def get_data_dtype(self, key):
        return str(numpy.asarray(self.data[0][key]).dtype)

    def have_corpus_seq_idx(self):
        return True

    def get_corpus_seq_idx(self, seq_idx):
        return self._seq_order[seq_idx]

    def have_get_corpus_seq(self):
        return True

    def get_corpus_seq(self, corpus_seq_idx):
        d = self.data[corpus_seq_idx]
        return DatasetSeq(seq_idx=corpus_seq_idx, features={k: numpy.asarray(v) for k, v in d.items() if k != "seq_tag"},
                          seq_tag=d.get("seq_tag", "seq-%i" % corpus_seq_idx))

    def get_current_seq_order(self):
        return self._seq_order


class CopyTaskDataset(GeneratingDataset):
    """
    Copy task: targets = inputs, random sparse labels. The length is uniform in ``[minlen, maxlen]``; both bounds can grow with the
    epoch (``*_epoch_factor``). Reference: returnn/datasets/generating.py:1231-1277.
    """

    def __init__(self, nsymbols: int, minlen: int = 0, maxlen: int = 0, minlen_epoch_factor: float = 0, maxlen_epoch_factor: float = 0,
                 minimum_size: Optional[int] = None, maximum_size: Optional[int] = None, **kwargs):
        super().__init__(input_dim=nsymbols, output_dim={"data": (nsymbols, 1), "classes": (nsymbols, 1)}, **kwargs)
        assert nsymbols <= 256
        self.nsymbols = nsymbols
        # minimum_size / maximum_size: the names this class used before it took over the reference's
        self.minlen = minlen if minimum_size is None else minimum_size
        self.maxlen = maxlen if maximum_size is None else maximum_size
        self.minlen_epoch_factor, self.maxlen_epoch_factor = minlen_epoch_factor, maxlen_epoch_factor

    def get_random_seq_len(self) -> int:
        """uniform in the epoch's [min, max]"""
        epoch = self.epoch or 1
        lo = int(self.minlen + self.minlen_epoch_factor * epoch)
        hi = int(self.maxlen + self.maxlen_epoch_factor * epoch)
        assert 0 < lo <= hi, "CopyTaskDataset: need 0 < minlen <= maxlen, got %i, %i" % (lo, hi)
        return self.random.randint(lo, hi + 1)

    def generate_seq(self, seq_idx: int) -> DatasetSeq:
        seq = numpy.array([self.random.randint(0, self.nsymbols) for _ in range(self.get_random_seq_len())], dtype="int8")
        return DatasetSeq(seq_idx=seq_idx, features=seq, targets={"classes": seq})


# The corpus readers live in their own module; the reference has them in its generating module
# (returnn/datasets/generating.py: LibriSpeechCorpus, TimitDataset, BlissDataset, Enwik8Corpus), so configs name them through here.
from .corpora import LibriSpeechCorpus, TimitDataset, NltkTimitDataset, BlissDataset, Enwik8Corpus  # noqa: E402

__all__ += ["LibriSpeechCorpus", "TimitDataset", "BlissDataset", "Enwik8Corpus"]
