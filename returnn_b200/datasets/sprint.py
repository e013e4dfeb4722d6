"""
Datasets fed by an external feature producer (RASR, historically "Sprint").

:class:`SprintDatasetBase` is a bounded producer / consumer window over sequences: a producer thread (the RASR process
embedding Python, or the reader thread of :class:`ExternSprintDataset`) pushes sequences with :meth:`add_new_data`, the
training thread pulls them through the ordinary dataset interface (``load_seqs`` / ``get_data``). Neither the number of
sequences nor the number of frames of an epoch is known before the producer says that the epoch is over, so ``num_seqs``
blocks until then and ``is_less_than_num_seqs`` answers from what has arrived.

:class:`ExternSprintDataset` starts the producer as a child process, passes it two pipe descriptors on its command line and reads
length-prefixed pickled messages from it (``("init", input_dim, output_dim, num_segments)``, ``("data", tag, features,
targets)``, ``("exit",)``); the Python side running inside that child is :mod:`returnn_b200.sprint.extern_interface`.

Parity: returnn/datasets/sprint.py (SprintDatasetBase :32, ExternSprintDataset :658). ``SprintCacheDataset`` (reader of RASR
feature / alignment archives) is not part of this module.
"""

from __future__ import annotations
import atexit
import os
import pickle
import struct
import subprocess
import threading
from typing import Any, Callable, Dict, List, Optional, Sequence, Union
import numpy

from .basic import Dataset, DatasetSeq
from ..log import log


class SprintDatasetBase(Dataset):
    """window over the sequences a producer thread pushes; see the module docstring"""

    # the producer is held back once it is this far ahead of the consumer, and released again at the lower mark
    SprintCachedSeqsMax = 200
    SprintCachedSeqsMin = 100

    def __init__(self, target_maps: Optional[Dict[str, Union[str, Dict[str, int]]]] = None, str_add_final_zero: bool = False,
                 input_stddev: float = 1.0, orth_post_process: Union[None, str, Sequence[str], Callable[[str], str]] = None,
                 bpe: Optional[Dict[str, Any]] = None, orth_vocab: Optional[Dict[str, Any]] = None,
                 suppress_load_seqs_print: bool = False, reduce_target_factor: int = 1, **kwargs):
        """
        :param target_maps: ``{key: file or dict}``: the string target ``key`` (e.g. "speaker_name") becomes the index of its line in the
            file; a scalar result is repeated over the frames
        :param str_add_final_zero: string targets additionally appear as ``key + "0"`` with a trailing zero byte
        :param input_stddev: features are divided by this
        :param orth_post_process: function(s) applied to the "orth" target (names as for ``LmDataset``)
        :param bpe: options of ``BytePairEncoding``: adds the target "bpe" computed from "orth"
        :param orth_vocab: options of ``Vocabulary.create_vocab``: adds the target "orth_classes" computed from "orth"
        :param suppress_load_seqs_print: no log line per ``load_seqs``
        :param reduce_target_factor: the alignment ("classes") has ceil(frames / factor) entries
        """
        super().__init__(**kwargs)
        assert isinstance(reduce_target_factor, int) and reduce_target_factor >= 1
        assert self.shuffle_frames_of_nseqs == 0, "%s: frames are shuffled by the producer, not here" % self
        self.suppress_load_seqs_print = suppress_load_seqs_print
        self.reduce_target_factor = reduce_target_factor
        self.str_add_final_zero = str_add_final_zero
        self.input_stddev = input_stddev
        self.target_maps: Optional[Dict[str, Dict[str, int]]] = None
        if target_maps:
            self.target_maps = {}
            for key, m in target_maps.items():
                if isinstance(m, str):
                    with open(m) as f:
                        m = {line: i for i, line in enumerate(f.read().splitlines())}
                assert isinstance(m, dict)
                self.target_maps[key] = m
        self.labels["orth"] = [chr(i) for i in range(255)]  # "orth" is the utf8 byte string
        self.orth_post_process: Optional[Callable[[str], str]] = None
        if orth_post_process:
            if callable(orth_post_process):
                self.orth_post_process = orth_post_process
            else:
                from .lm import get_post_processor_function

                self.orth_post_process = get_post_processor_function(orth_post_process)
        self.bpe = None
        if bpe:
            from .util.vocabulary import BytePairEncoding, Vocabulary

            self.bpe = bpe if isinstance(bpe, Vocabulary) else BytePairEncoding(**bpe)
            self.labels["bpe"] = self.bpe.labels
        self.orth_vocab = None
        if orth_vocab:
            from .util.vocabulary import Vocabulary

            self.orth_vocab = orth_vocab if isinstance(orth_vocab, Vocabulary) else Vocabulary.create_vocab(**orth_vocab)
            self.labels["orth_classes"] = self.orth_vocab.labels
        self._cond = threading.Condition(threading.RLock())
        self.multiple_epochs = False
        self.sprint_epoch: Optional[int] = None  # epoch the producer is in
        self.returnn_epoch: Optional[int] = None  # epoch the consumer asked for
        self.sprint_finalized = False
        self.predefined_seq_list_order: Optional[List[str]] = None
        self._dropped_target_keys: List[str] = []
        self._complete_frac: Optional[float] = None
        self._window_reset()

    # -- state of one epoch --------------------------------------------------------------------------------------------
    def _window_reset(self):
        self._seqs: List[DatasetSeq] = []  # consecutive sequence indices, the oldest ones dropped once the consumer moved on
        self._next_idx = 0  # index the next pushed sequence gets
        self._wanted_end = 0  # end of the last range the consumer asked for
        self._epoch_open = False  # the producer may push
        self._epoch_done = False  # the producer said that the epoch is over
        self._epoch_seen_all = False
        self._num_timesteps = 0
        self._complete_frac = None

    def use_multiple_epochs(self):
        """the producer goes through several epochs itself (it calls :meth:`init_sprint_epoch` for each)"""
        self.multiple_epochs = True

    def set_dimensions(self, input_dim: int, output_dim: int):
        """called by the producer side once the feature and label dimensions are known"""
        assert input_dim > 0
        self.num_inputs = input_dim
        self.num_outputs = {"data": (input_dim * self.window, 2)}
        if output_dim > 0:
            self.num_outputs["classes"] = (output_dim, 1)
        if self.bpe:
            self.num_outputs["bpe"] = (self.bpe.num_labels, 1)
        if self.orth_vocab:
            self.num_outputs["orth_classes"] = (self.orth_vocab.num_labels, 1)
        self.num_outputs["orth"] = (256, 1)
        self._base_init()
        with self._cond:
            if not self._epoch_open:  # a producer that took its segment order from here has opened the epoch before it knows the dimensions
                self._window_reset()

    def initialize(self):
        """no epoch-less first order here: :meth:`init_seq_order` waits for the producer, which may be the very thread that calls this"""
        self._base_init()

    # -- producer side ---------------------------------------------------------------------------------------------------
    def init_sprint_epoch(self, epoch: Optional[int]):
        """the producer starts (its view of) an epoch; from now on it may push"""
        with self._cond:
            self.sprint_epoch = epoch
            self.sprint_finalized = False
            self._window_reset()
            self._epoch_open = True
            self._cond.notify_all()

    def finalize_sprint(self):
        """the producer is gone for good"""
        with self._cond:
            self.sprint_finalized = True
            self._cond.notify_all()

    def finish_sprint_epoch(self, seen_all: bool = True):
        """the producer has no more sequences for this epoch"""
        with self._cond:
            self._epoch_done = True
            self._epoch_seen_all = seen_all
            self._epoch_open = False
            self._cond.notify_all()

    def wait_for_returnn_epoch(self, epoch: int):
        """producer side, with :meth:`use_multiple_epochs`: block until the consumer has asked for ``epoch``"""
        with self._cond:
            while self.returnn_epoch != epoch:
                assert self.returnn_epoch is None or self.returnn_epoch <= epoch, "%s: consumer is at epoch %r, producer at %r" % (
                    self, self.returnn_epoch, epoch)
                self._cond.wait()

    def _convert_targets(self, targets: Dict[str, Any], num_frames: int) -> Dict[str, numpy.ndarray]:
        if "speaker_name" in targets:
            targets["speaker_name"] = targets["speaker_name"].strip()
        if "orth" in targets:
            orth = targets["orth"].strip()
            targets["orth"] = self.orth_post_process(orth) if self.orth_post_process else orth
        if self.bpe:
            assert isinstance(targets.get("orth"), str) and "bpe" not in targets
            targets["bpe"] = numpy.array(self.bpe.get_seq(targets["orth"]), dtype="int32")
        if self.orth_vocab:
            assert isinstance(targets.get("orth"), str) and "orth_classes" not in targets
            targets["orth_classes"] = numpy.array(self.orth_vocab.get_seq(targets["orth"]), dtype="int32")
        for key, mapping in (self.target_maps or {}).items():
            assert key in targets, "%s: target_maps key %r not delivered by the producer" % (self, key)
            v = numpy.asarray(mapping[targets[key]])
            targets[key] = numpy.full((num_frames,), v, dtype=v.dtype) if v.ndim == 0 else v
        out: Dict[str, numpy.ndarray] = {}
        for key in sorted(targets):
            if key in self._dropped_target_keys:
                continue
            v = targets[key]
            if isinstance(v, str):
                v = v.encode("utf8")
            if isinstance(v, bytes):
                arr = numpy.frombuffer(v, dtype="uint8").copy()
                out[key] = arr
                if self.str_add_final_zero:
                    assert key + "0" not in targets
                    out[key + "0"] = numpy.append(arr, numpy.zeros(1, dtype="uint8"))
            elif isinstance(v, numpy.ndarray):
                out[key] = v
            else:
                print("%s: target %r is not an array (%r), ignored from now on" % (self, key, type(v)), file=log.v3)
                self._dropped_target_keys.append(key)
        return out

    def add_new_data(self, features: numpy.ndarray, targets=None, segment_name: Optional[str] = None) -> int:
        """
        Producer side: one more sequence.

        :param features: [feature, time], as RASR hands them over
        :param targets: dict key -> array / string, or the alignment [time] alone (key "classes")
        :param segment_name: tag
        :return: index of the sequence within the epoch
        """
        assert features.shape[0] == self.num_inputs, "%s: got %i features, expected %i" % (self, features.shape[0], self.num_inputs)
        num_frames = features.shape[1]
        feats = numpy.ascontiguousarray(features.T)
        if self.input_stddev != 1:
            feats = feats / self.input_stddev
        if self.window > 1:
            feats = self._sliding_window(feats)
        if targets is None:
            targets = {}
        elif not isinstance(targets, dict):
            targets = {"classes": targets}
        else:
            targets = dict(targets)
        if "classes" in targets:
            want = -(-num_frames // self.reduce_target_factor)
            assert targets["classes"].shape == (want,), "%s: alignment of %r entries for %i frames (reduce_target_factor %i)" % (
                self, targets["classes"].shape, num_frames, self.reduce_target_factor)
        arrays = self._convert_targets(targets, num_frames)
        with self._cond:
            assert self._epoch_open and not self._epoch_done and not self.sprint_finalized, "%s: add_new_data outside of an epoch" % self
            idx = self._next_idx
            if self.predefined_seq_list_order:
                assert idx < len(self.predefined_seq_list_order), "%s: sequence %i beyond the %i expected ones" % (
                    self, idx, len(self.predefined_seq_list_order))
                want_tag = self.predefined_seq_list_order[idx]
                if want_tag != segment_name:
                    where = self.predefined_seq_list_order.index(segment_name) if segment_name in self.predefined_seq_list_order else None
                    raise Exception("%s: sequence %i should be %r but the producer sent %r (%s)" % (
                        self, idx, want_tag, segment_name, ("which is expected at index %i" % where) if where is not None else "not in the list"))
            self._next_idx += 1
            self._num_timesteps += num_frames
            self._cond.notify_all()
            if idx >= self._wanted_end + self.SprintCachedSeqsMax:
                while idx >= self._wanted_end + self.SprintCachedSeqsMin and not self.sprint_finalized:
                    self._cond.wait()
            self._seqs.append(DatasetSeq(idx, feats, targets=arrays, seq_tag=segment_name))
            self._cond.notify_all()
            return idx

    # -- consumer side ---------------------------------------------------------------------------------------------------
    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        """
        The order is the producer's; only a ``seq_list`` to check the arriving tags against can be given.
        Blocks until the producer has opened an epoch.
        """
        assert seq_order is None, "%s: the producer defines the order" % self
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        with self._cond:
            self.returnn_epoch = epoch
            self.predefined_seq_list_order = list(seq_list) if seq_list is not None else None
            self._cond.notify_all()
            # a producer that walks the epochs itself waits for this call and then opens the epoch: the window of its previous epoch
            # (finished, hence "done") must not be taken for the new one
            while not ((self._epoch_open or self._epoch_done) and (not self.multiple_epochs or not epoch or (self.sprint_epoch or 0) >= epoch)) and not self.sprint_finalized:
                self._cond.wait()
            self._wanted_end = 0
        return True

    def _first_idx(self) -> int:
        return self._seqs[0].seq_idx if self._seqs else self._next_idx

    def _arrived(self, idx: int) -> bool:
        return bool(self._seqs) and idx <= self._seqs[-1].seq_idx

    def _wait_for(self, idx: int) -> bool:
        """until sequence ``idx`` has arrived; False if the epoch ended before"""
        with self._cond:
            while True:
                if self._arrived(idx):
                    return True
                if self._epoch_done or self.sprint_finalized:
                    return False
                self._cond.wait()

    def is_cached(self, start, end):
        with self._cond:
            if start >= end:
                return True
            return self._seqs and self._first_idx() <= start and self._arrived(end - 1)

    def _load_seqs(self, start, end):
        if not self.suppress_load_seqs_print:
            print("%s load_seqs in %s: [%i, %i)" % (self, threading.current_thread().name, start, end), file=log.v5)
        with self._cond:
            self._wanted_end = max(self._wanted_end, end)
            while self._seqs and self._seqs[0].seq_idx < start:  # the consumer only moves forward
                self._seqs.pop(0)
            self._cond.notify_all()
        if end > start:
            self._wait_for(end - 1)

    def _seq(self, idx: int) -> DatasetSeq:
        with self._cond:
            assert self._wait_for(idx), "%s: sequence %i does not exist (the epoch has %i)" % (self, idx, self._next_idx)
            first = self._first_idx()
            assert idx >= first, "%s: sequence %i was already dropped (window starts at %i)" % (self, idx, first)
            return self._seqs[idx - first]

    def load_seqs(self, start, end):
        """always goes through :meth:`_load_seqs`: the consumer's position is what releases the producer, also for cached ranges"""
        assert 0 <= start <= end
        if start == end:
            return
        self._load_seqs(start, end)

    def get_num_timesteps(self):
        """frames so far (final once the epoch is over)"""
        with self._cond:
            return self._num_timesteps

    @property
    def num_seqs(self):
        """blocks until the producer has finished the epoch"""
        with self._cond:
            if self.predefined_seq_list_order:
                return len(self.predefined_seq_list_order)
            while not self._epoch_done and not self.sprint_finalized:
                self._cond.wait()
            return self._next_idx

    def have_seqs(self) -> bool:
        """whether the epoch has at least one sequence"""
        return self.is_less_than_num_seqs(0)

    def is_less_than_num_seqs(self, n):
        if n < 0:
            return True
        return self._wait_for(n)

    def get_data_keys(self):
        keys = ["data"] + self.get_target_list()
        return keys

    def get_target_list(self):
        with self._cond:
            if self._seqs:
                return sorted(k for k in self._seqs[0].features.keys() if k != "data")
        return sorted(k for k in self.num_outputs.keys() if k != "data") if self.num_outputs else []

    def set_complete_frac(self, frac: float):
        """the producer knows how far it is"""
        self._complete_frac = frac

    def get_complete_frac(self, sorted_seq_idx, **kwargs):
        with self._cond:
            if self.predefined_seq_list_order:
                return self.generic_complete_frac(sorted_seq_idx, len(self.predefined_seq_list_order))
            if self._epoch_done:
                return self.generic_complete_frac(sorted_seq_idx, self._next_idx)
            if self._complete_frac is not None:
                return self._complete_frac
            return self.generic_complete_frac(sorted_seq_idx, None)

    def get_seq_length(self, sorted_seq_idx):
        return self._seq(sorted_seq_idx).num_frames

    def get_data(self, seq_idx, key):
        return self._seq(seq_idx).features[key]

    def get_input_data(self, sorted_seq_idx):
        return self.get_data(sorted_seq_idx, "data")

    def get_targets(self, target, sorted_seq_idx):
        return self._seq(sorted_seq_idx).features.get(target)

    def get_tag(self, sorted_seq_idx):
        return self._seq(sorted_seq_idx).seq_tag


def _read_msg(fd_file):
    """one length-prefixed pickled message or None at end of stream"""
    head = fd_file.read(8)
    if len(head) < 8:
        return None
    (n,) = struct.unpack("<Q", head)
    body = fd_file.read(n)
    if len(body) < n:
        return None
    return pickle.loads(body)


def write_msg(fd_file, obj):
    """counterpart of the reader above (used by the producer side)"""
    body = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    fd_file.write(struct.pack("<Q", len(body)))
    fd_file.write(body)
    fd_file.flush()


class ExternSprintDataset(SprintDatasetBase):
    """
    The producer runs as a child process: ``sprintTrainerExecPath`` with ``sprintConfigStr`` plus the options that make it load
    :mod:`returnn_b200.sprint.extern_interface` and tell it the two pipe descriptors. One child per epoch; a reader thread feeds what
    it sends into :meth:`add_new_data`.
    """

    def __init__(self, sprintTrainerExecPath: Union[str, Sequence[str]], sprintConfigStr: Union[str, Sequence[str], Callable[[], str]] = "",
                 partitionEpoch: Optional[int] = None, **kwargs):
        """
        :param sprintTrainerExecPath: executable (or argv prefix) of the producer
        :param sprintConfigStr: further command-line options, a string (split at blanks), a list, or a function returning either
        :param partitionEpoch: deprecated spelling of ``partition_epoch``
        """
        super().__init__(**kwargs)
        self.sprintTrainerExecPath = sprintTrainerExecPath
        self.sprintConfig = sprintConfigStr
        if partitionEpoch:
            assert self.partition_epoch == 1, "%s: give only one of partitionEpoch / partition_epoch" % self
            self.partition_epoch = partitionEpoch
        self._child: Optional[subprocess.Popen] = None
        self._reader: Optional[threading.Thread] = None
        self._from_child = None
        self._to_child = None
        self._estimated_num_seqs: Optional[int] = None
        self._reader_error: Optional[BaseException] = None
        self.seq_list_file: Optional[str] = None
        atexit.register(self._stop_child)
        # one short-lived child tells the dimensions
        self._start_child(epoch=None, dims_only=True)

    def _argv(self, epoch: Optional[int], c2p_w: int, p2c_r: int) -> List[str]:
        exe = self.sprintTrainerExecPath
        argv = [exe] if isinstance(exe, str) else list(exe)
        cfg = self.sprintConfig() if callable(self.sprintConfig) else self.sprintConfig
        argv += cfg.split() if isinstance(cfg, str) else list(cfg)
        opts = ["action:ExternSprintDataset", "c2p_fd:%i" % c2p_w, "p2c_fd:%i" % p2c_r]
        pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        argv += [
            "--*.seed=%i" % ((epoch or 1) // self.partition_epoch),
            "--*.python-segment-order=true", "--*.python-segment-order-pymod-path=%s" % pkg_parent,
            "--*.python-segment-order-pymod-name=returnn_b200.sprint.extern_interface",
            "--*.use-data-source=false", "--*.trainer=python-trainer", "--*.pymod-path=%s" % pkg_parent,
            "--*.pymod-name=returnn_b200.sprint.extern_interface", "--*.pymod-config=%s" % ",".join(opts),
        ]
        if self.partition_epoch > 1:
            argv += ["--*.corpus.partition=%i" % self.partition_epoch, "--*.corpus.select-partition=%i" % (((epoch or 1) - 1) % self.partition_epoch)]
        if self.seq_list_file:
            argv += ["--*.corpus.segment-order-shuffle=false", "--*.corpus.segments.file=%s" % self.seq_list_file,
                     "--*.corpus.segment-order=%s" % self.seq_list_file]
        return argv

    def _start_child(self, epoch: Optional[int], dims_only: bool = False):
        self._stop_child()
        c2p_r, c2p_w = os.pipe()
        p2c_r, p2c_w = os.pipe()
        argv = self._argv(epoch, c2p_w, p2c_r)
        print("%s: starting producer: %s" % (self, " ".join(argv)), file=log.v5)
        self._child = subprocess.Popen(argv, pass_fds=(c2p_w, p2c_r), stdin=subprocess.DEVNULL)
        os.close(c2p_w)
        os.close(p2c_r)
        self._from_child = os.fdopen(c2p_r, "rb")
        self._to_child = os.fdopen(p2c_w, "wb")
        msg = _read_msg(self._from_child)
        if msg is None or msg[0] != "init":
            code = self._child.wait()
            self._stop_child()
            raise Exception("%s: the producer did not announce itself (exit code %r, first message %r)" % (self, code, msg))
        _, input_dim, output_dim, num_segments = msg
        if dims_only:
            self.set_dimensions(input_dim, output_dim)
            self._estimated_num_seqs = num_segments
            self._stop_child()
            return
        self._estimated_num_seqs = num_segments
        self.init_sprint_epoch(epoch)
        self._reader_error = None
        self._reader = threading.Thread(target=self._reader_loop, args=(self._child, self._from_child), name="%s reader" % self.name, daemon=True)
        self._reader.start()

    def _reader_loop(self, child: subprocess.Popen, stream):
        seen_all = False
        try:
            while True:
                msg = _read_msg(stream)
                if msg is None:
                    break
                if msg[0] == "data":
                    _, tag, features, targets = msg
                    self.add_new_data(numpy.asarray(features), targets, segment_name=tag)
                elif msg[0] == "exit":
                    seen_all = True
                    break
                else:
                    raise Exception("%s: unknown message %r from the producer" % (self, msg[0]))
        except BaseException as exc:  # handed to the consumer: it would wait forever otherwise
            self._reader_error = exc
        finally:
            if child is self._child:
                self.finish_sprint_epoch(seen_all=seen_all)

    def _stop_child(self):
        child, self._child = self._child, None
        for f in (self._to_child, self._from_child):
            try:
                if f is not None:
                    f.close()
            except Exception:
                pass
        self._to_child = self._from_child = None
        if child is not None:
            with self._cond:
                self.sprint_finalized = True  # releases a reader that is held back in add_new_data
                self._cond.notify_all()
            try:
                child.wait(timeout=5)
            except subprocess.TimeoutExpired:
                child.terminate()
                try:
                    child.wait(timeout=5)
                except subprocess.TimeoutExpired:
                    child.kill()
                    child.wait()
        reader, self._reader = self._reader, None
        if reader is not None and reader is not threading.current_thread():
            reader.join(timeout=10)

    def _wait_for(self, idx):
        res = super()._wait_for(idx)
        if self._reader_error is not None:
            raise Exception("%s: reading from the producer failed" % self) from self._reader_error
        return res

    @property
    def estimated_num_seqs(self):
        """what the producer announced"""
        return self._estimated_num_seqs

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        assert seq_order is None
        if seq_list is not None:
            import tempfile

            with tempfile.NamedTemporaryFile("w", prefix="returnn-seq-list-", suffix=".txt", delete=False) as f:
                f.write("\n".join(seq_list) + "\n")
            self.seq_list_file = f.name
        else:
            self.seq_list_file = None
        self._start_child(epoch)
        return super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=None)

    def finish_epoch(self, *, free_resources: bool = False):
        super().finish_epoch(free_resources=free_resources)
        self._stop_child()
        if self.seq_list_file:
            try:
                os.unlink(self.seq_list_file)
            except OSError:
                pass
            self.seq_list_file = None

    def __del__(self):
        try:
            self._stop_child()
        except Exception:
            pass


class SprintCacheDataset(Dataset):
    """
    Reads Sprint archives (single files or bundles) directly: feature caches as float32 ``[T, D]`` and alignment caches as class
    labels ``[T]`` (mapped through an allophone labeling: state tying or phoneme list). No RASR process is involved.

    ``data`` maps a data key to reader options: ``{"data": {"filename": "features.cache"}, "classes": {"filename": "align.cache",
    "allophone_labeling": {"silence_phone": "si", "allophone_file": ..., "state_tying_file": ...}}}``; the type ("feat" / "align") is
    taken from the key or from the presence of ``allophone_labeling`` unless ``data_type`` names it.

    Every key must hold the same entry names; the sequence order (sorting by entry size) works from the table of contents alone.

    Parity: returnn/datasets/sprint.py (``SprintCacheDataset`` :1064, its ``SprintCacheReader`` :1071).
    """

    class SprintCacheReader:
        """one archive (or bundle) behind one data key"""

        def __init__(self, data_key: str, filename: str, data_type: Optional[str] = None, allophone_labeling: Optional[dict] = None):
            from ..sprint.cache import open_file_archive, AllophoneLabeling

            self.data_key = data_key
            self.sprint_cache = open_file_archive(filename)
            if not data_type:
                data_type = {"data": "feat", "classes": "align"}.get(data_key, "align" if allophone_labeling else "feat")
            assert data_type in ("feat", "align"), "%r: data_type %r" % (data_key, data_type)
            self.type = data_type
            self.allophone_labeling = None
            if allophone_labeling:
                self.allophone_labeling = AllophoneLabeling(**allophone_labeling)
                self.sprint_cache.set_allophones(self.allophone_labeling.allophone_file)
            else:
                assert data_type != "align", "%r: an alignment needs allophone_labeling" % data_key
            self.content_keys = [name for name in self.sprint_cache.file_list() if not name.endswith(".attribs")]
            if data_type == "align":
                self.num_labels = self.allophone_labeling.num_labels
                self.dtype = "int8" if self.num_labels < 2**7 else "int16" if self.num_labels < 2**15 else "int32"
                self.num_dims = 1
                if self.allophone_labeling.state_tying_by_allo_state_idx:
                    self.type = "align_raw"  # the tying is keyed by the undivided emission index: no split per frame
            else:
                assert self.content_keys, "%r: empty feature cache %r" % (data_key, filename)
                _, feats = self.sprint_cache.read(self.content_keys[0], "feat")
                assert len(feats) > 0 and feats[0].ndim == 1
                self.num_labels = int(feats[0].shape[0])
                self.num_dims = 2
                self.dtype = "float32"

        def read(self, name: str) -> numpy.ndarray:
            """:return: ``[T, D]`` features or ``[T]`` labels of the entry"""
            res = self.sprint_cache.read(name, typ=self.type)
            if self.type == "feat":
                times, feats = res
                mat = numpy.asarray(feats, dtype=self.dtype)
                assert mat.shape == (len(times), self.num_labels), "%r: entry %r has shape %r" % (self.data_key, name, mat.shape)
                return mat
            assert all(w == 1 for (_, _, _, w) in res), "%r: entry %r is a soft alignment, which is not supported" % (self.data_key, name)
            if self.type == "align_raw":
                tying = self.allophone_labeling.state_tying_by_allo_state_idx
                return numpy.array([tying[e] for (_, e, _, _) in res], dtype=self.dtype)
            label = self.allophone_labeling.get_label_idx
            return numpy.array([label(a, s) for (_, a, s, _) in res], dtype=self.dtype)

    def __init__(self, data: Dict[str, dict], **kwargs):
        super().__init__(**kwargs)
        self.data = {key: self.SprintCacheReader(data_key=key, **opts) for key, opts in data.items()}
        assert "data" in self.data, "%s: needs the key 'data'" % self
        self.seq_list_original = list(self.data["data"].content_keys)
        self.seq_list_ordered = self.seq_list_original
        names = sorted(self.seq_list_original)
        for key, reader in self.data.items():
            assert sorted(reader.content_keys) == names, "%s: the entries of %r differ from those of 'data'" % (self, key)
        self.num_outputs = {key: (r.num_labels, r.num_dims) for key, r in self.data.items()}
        self.num_inputs = self.num_outputs["data"][0]
        self._num_seqs = len(self.seq_list_original)
        self._loaded: Dict[int, DatasetSeq] = {}
        self.epoch = None

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        assert seq_list is None and seq_order is None, "%s: no predefined order" % self
        again = self.epoch is None or self.epoch != epoch
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        self.epoch = epoch
        if not again:
            return False
        toc = self.data["data"].sprint_cache.ft
        order = self.get_seq_order_for_epoch(epoch, num_seqs=len(self.seq_list_original), get_seq_len=lambda i: toc[self.seq_list_original[i]].size)
        self.seq_list_ordered = [self.seq_list_original[i] for i in order]
        self._num_seqs = len(self.seq_list_ordered)
        self._loaded.clear()
        return True

    @property
    def num_seqs(self) -> int:
        return self._num_seqs

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self.seq_list_original)

    def get_all_tags(self) -> List[str]:
        return list(self.seq_list_original)

    def supports_seq_order_sorting(self) -> bool:
        return True

    def supports_sharding(self) -> bool:
        return True

    def get_dataset_seq_for_name(self, name: str, seq_idx: int = -1) -> DatasetSeq:
        """:return: the sequence of this entry name, all keys read"""
        return DatasetSeq(seq_idx=seq_idx, seq_tag=name, features={key: r.read(name) for key, r in self.data.items()})

    def is_cached(self, start, end):
        return False

    def _load_seqs(self, start: int, end: int):
        for i in [i for i in self._loaded if i < start]:
            del self._loaded[i]
        for i in range(start, min(end, self._num_seqs)):
            if i not in self._loaded:
                self._loaded[i] = self.get_dataset_seq_for_name(self.seq_list_ordered[i], seq_idx=i)

    def _seq(self, seq_idx: int) -> DatasetSeq:
        if seq_idx not in self._loaded:
            self._loaded[seq_idx] = self.get_dataset_seq_for_name(self.seq_list_ordered[seq_idx], seq_idx=seq_idx)
        return self._loaded[seq_idx]

    def get_seq_length(self, seq_idx: int):
        return self._seq(seq_idx).num_frames

    def get_data(self, seq_idx: int, key: str) -> numpy.ndarray:
        return self._seq(seq_idx).features[key]

    def get_input_data(self, seq_idx: int) -> numpy.ndarray:
        return self.get_data(seq_idx, "data")

    def get_targets(self, target: str, seq_idx: int) -> numpy.ndarray:
        return self.get_data(seq_idx, target)

    def get_data_keys(self) -> List[str]:
        return list(self.data.keys())

    def get_target_list(self) -> List[str]:
        return [key for key, r in self.data.items() if r.type != "feat"]

    def get_data_dtype(self, key: str) -> str:
        return self.data[key].dtype

    def get_tag(self, sorted_seq_idx: int) -> str:
        return self.seq_list_ordered[sorted_seq_idx]
