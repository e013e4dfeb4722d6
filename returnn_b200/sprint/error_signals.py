"""
Sequence-discriminative criteria computed by RASR ("Sprint") child processes: the trainer sends the (log) posteriors of a sequence,
RASR answers with the loss and its gradient (the "error signal"), and :func:`sprint_loss` ties that into autograd.

* :class:`SprintSubprocessInstance`: one RASR child. It is started with this package's ``sprint.control`` module as its
  PythonControl (``--*.pymod-name``), two pipes passed by descriptor number (``--*.pymod-config=c2p_fd:..,p2c_fd:..``), and speaks
  the length-prefixed-pickle protocol documented there.
* :class:`SprintInstancePool`: ``numInstances`` children per set of options. A batch is a work queue, longest sequences first; every
  child gets one sequence, and whichever answers first (``selectors`` on the answer pipes) gets the next. No thread per child and
  no static partition: a child that draws slow sequences simply takes fewer.
* :func:`sprint_loss`: ``[B, T, D]`` log posteriors + lengths + sequence tags -> ``[B]`` losses; the backward pass multiplies the
  stored error signal with the incoming gradient.
* :meth:`SprintInstancePool.get_automata_for_batch`: the allophone-state automata of a batch, merged into one edge list for the
  ``fast_baum_welch`` op.

Parity: returnn/sprint/error_signals.py (``SprintSubprocessInstance`` :25, ``SprintInstancePool`` :361).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple
import atexit
import os
import selectors
import subprocess
import threading
import numpy

from ..utils.basic import read_pickled_object, write_pickled_object


def _shell_args(v) -> List[str]:
    if callable(v):
        v = v()
    if isinstance(v, str):
        import shlex

        return shlex.split(v)
    return [str(x) for x in (v or [])]


class SprintSubprocessInstance:
    """
    One RASR child process.

    :param sprintExecPath: the RASR executable (e.g. ``nn-trainer``)
    :param minPythonControlVersion: checked inside the child against RASR's PythonControl version
    :param sprintConfigStr: further command line arguments; ``config:<key>`` looks the value up in the global config; a callable is
        called
    :param sprintControlConfig: further ``key:value`` entries for the child's ``--*.pymod-config``
    :param usePythonSegmentOrder: RASR takes its segment order from the commands (``--*.python-segment-order=true``)

    The argument names are the ones user configs use.
    """

    Version = 1  # of the pipe protocol

    def __init__(self, sprintExecPath: str, minPythonControlVersion: int = 2, sprintConfigStr="", sprintControlConfig: Optional[Dict[str, Any]] = None,
                 usePythonSegmentOrder: bool = True):
        assert os.path.exists(sprintExecPath), "RASR executable %r does not exist" % sprintExecPath
        self.sprintExecPath = sprintExecPath
        self.minPythonControlVersion = minPythonControlVersion
        if isinstance(sprintConfigStr, str) and sprintConfigStr.startswith("config:"):
            from ..config import get_global_config

            sprintConfigStr = get_global_config().typed_dict[sprintConfigStr[len("config:"):]]
        self.sprintConfig = _shell_args(sprintConfigStr)
        self.sprintControlConfig = dict(sprintControlConfig or {})
        self.usePythonSegmentOrder = usePythonSegmentOrder
        self.child: Optional[subprocess.Popen] = None
        self.parent_pid = os.getpid()
        self.is_calculating = False
        self._cur_seg_name = None
        self._cur_shape = None
        self._to_child = self._from_child = None
        atexit.register(self.exit_handler)
        self.init()

    # -- life cycle --

    def init(self):
        """(re)start the child and shake hands"""
        self._exit_child()
        self._start_child()

    def _build_sprint_args(self, c2p_fd: int, p2c_fd: int) -> List[str]:
        cfg = ["c2p_fd:%i" % c2p_fd, "p2c_fd:%i" % p2c_fd, "minPythonControlVersion:%i" % self.minPythonControlVersion]
        cfg += ["%s:%s" % kv for kv in sorted(self.sprintControlConfig.items())]
        cfg_str = ",".join(cfg)
        mod_path = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        mod_name = "returnn_b200.sprint.control"
        args = [self.sprintExecPath, "--*.python-control-enabled=true", "--*.pymod-path=%s" % mod_path, "--*.pymod-name=%s" % mod_name,
                "--*.pymod-config=%s" % cfg_str]
        if self.usePythonSegmentOrder:
            args += ["--*.python-segment-order=true", "--*.python-segment-order-pymod-path=%s" % mod_path,
                     "--*.python-segment-order-pymod-name=%s" % mod_name, "--*.python-segment-order-config=%s" % cfg_str,
                     "--*.python-segment-order-allow-copy=false"]
        return args + self.sprintConfig

    def _start_child(self):
        c2p_r, c2p_w = os.pipe()
        p2c_r, p2c_w = os.pipe()
        args = self._build_sprint_args(c2p_fd=c2p_w, p2c_fd=p2c_r)
        self.child = subprocess.Popen(args, pass_fds=(c2p_w, p2c_r), close_fds=True)
        os.close(c2p_w)
        os.close(p2c_r)
        self._from_child = os.fdopen(c2p_r, "rb")
        self._to_child = os.fdopen(p2c_w, "wb")
        self.is_calculating = False
        try:
            self._send(("init", "SprintSubprocessInstance", self.Version))
            ret = self._read()
            assert ret[0] == "ok" and len(ret) == 3 and ret[2] == self.Version, "unexpected answer to init: %r" % (ret,)
        except Exception:
            self._exit_child(interrupt=True)
            raise

    def _exit_child(self, interrupt: bool = False):
        if self.child is None:
            return
        try:
            if self.child.poll() is None and self._to_child is not None and not self._to_child.closed:
                if interrupt and self.is_calculating:
                    self.child.terminate()
                else:
                    try:
                        self._send(("exit",))
                    except (OSError, ValueError):
                        pass
        finally:
            for p in (self._to_child, self._from_child):
                try:
                    if p is not None:
                        p.close()
                except OSError:
                    pass
            try:
                self.child.wait(timeout=10)
            except subprocess.TimeoutExpired:
                self.child.kill()
                self.child.wait()
            self.child = None
            self._to_child = self._from_child = None
            self.is_calculating = False

    def exit_handler(self):
        """at interpreter exit (and from :meth:`SprintInstancePool.close`)"""
        if os.getpid() == self.parent_pid:
            self._exit_child(interrupt=True)

    # -- the pipe --

    def _send(self, v):
        assert os.getpid() == self.parent_pid
        write_pickled_object(self._to_child, v)

    def _read(self):
        assert os.getpid() == self.parent_pid
        return read_pickled_object(self._from_child)

    def fileno(self) -> int:
        """of the answer pipe, for ``select``"""
        return self._from_child.fileno()

    def _poll(self) -> bool:
        import select

        return bool(select.select([self.fileno()], [], [], 0)[0])

    # -- commands --

    def get_loss_and_error_signal__send(self, seg_name: str, seg_len: int, log_posteriors: numpy.ndarray):
        """:param log_posteriors: [T, D]; the answer is fetched with :meth:`get_loss_and_error_signal__read`"""
        assert not self.is_calculating and seg_name
        assert int(seg_len) == log_posteriors.shape[0]
        self._cur_seg_name, self._cur_shape = seg_name, log_posteriors.shape
        self._send(("get_loss_and_error_signal", seg_name, int(seg_len), numpy.ascontiguousarray(log_posteriors, dtype="float32")))
        self.is_calculating = True

    def get_loss_and_error_signal__have_data(self) -> bool:
        """whether the answer can be read without waiting"""
        assert self.is_calculating
        return self._poll()

    def get_loss_and_error_signal__read(self) -> Tuple[str, float, numpy.ndarray]:
        """:return: (segment name, loss, error signal [T, D])"""
        assert self.is_calculating
        ret = self._read()
        self.is_calculating = False
        if ret[0] != "ok":
            raise RuntimeError("RASR child failed on segment %r: %s" % (self._cur_seg_name, ret[1:]))
        assert len(ret) == 3, "unexpected answer: %r" % (ret,)
        loss, err = ret[1], ret[2]
        assert err.shape == self._cur_shape
        return self._cur_seg_name, loss, err

    def get_loss_and_error_signal(self, seg_name: str, seg_len: int, log_posteriors: numpy.ndarray) -> Tuple[float, numpy.ndarray]:
        """send and wait"""
        self.get_loss_and_error_signal__send(seg_name, seg_len, log_posteriors)
        _, loss, err = self.get_loss_and_error_signal__read()
        return loss, err

    def export_allophone_state_fsa_by_segment_name(self, segment_name: str):
        """:return: (num_states, num_edges, edges [3 * num_edges] uint32 as (from.., to.., emission..), weights [num_edges] float32)"""
        self._send(("export_allophone_state_fsa_by_segment_name", segment_name))
        ret = self._read()
        if ret[0] != "ok":
            raise RuntimeError("RASR child failed on the automaton of %r: %s" % (segment_name, ret[1:]))
        return ret[1:]


def _hashable(v):
    if isinstance(v, dict):
        return tuple(sorted((k, _hashable(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_hashable(x) for x in v)
    return v


class SprintInstancePool:
    """``numInstances`` children for one set of options (the other options go to :class:`SprintSubprocessInstance`)"""

    class_lock = threading.RLock()
    global_instances: Dict[Any, "SprintInstancePool"] = {}

    @classmethod
    def get_global_instance(cls, sprint_opts: Dict[str, Any]) -> "SprintInstancePool":
        """one pool per distinct options"""
        key = _hashable(sprint_opts)
        with cls.class_lock:
            if key not in cls.global_instances:
                cls.global_instances[key] = SprintInstancePool(sprint_opts)
            return cls.global_instances[key]

    def __init__(self, sprint_opts: Dict[str, Any]):
        self.lock = threading.RLock()  # callers from several threads take it themselves
        opts = dict(sprint_opts)
        self.max_num_instances = int(opts.pop("numInstances", 1))
        self.sprint_opts = opts
        self.instances: List[SprintSubprocessInstance] = []

    def _get_instance(self, i: int) -> SprintSubprocessInstance:
        assert i < self.max_num_instances
        while len(self.instances) <= i:
            self.instances.append(SprintSubprocessInstance(**self.sprint_opts))
        return self.instances[i]

    def get_free_instance(self) -> Optional[SprintSubprocessInstance]:
        """an idle child, a new one while the pool may grow, else None"""
        for inst in self.instances:
            if not inst.is_calculating:
                return inst
        if len(self.instances) < self.max_num_instances:
            return self._get_instance(len(self.instances))
        return None

    def close(self):
        """end all children"""
        for inst in self.instances:
            inst.exit_handler()
        self.instances = []

    def get_batch_loss_and_error_signal(self, log_posteriors: numpy.ndarray, seq_lengths: numpy.ndarray, tags: Sequence[str]) -> Tuple[numpy.ndarray, numpy.ndarray]:
        """
        :param log_posteriors: [T, B, D]
        :param seq_lengths: [B]
        :param tags: B sequence names as RASR's corpus knows them
        :return: loss [B], error signal [T, B, D] (zero beyond each sequence's length)
        """
        assert log_posteriors.ndim == 3 and seq_lengths.ndim == 1 and len(tags) == seq_lengths.shape[0] == log_posteriors.shape[1]
        n_batch = len(tags)
        loss = numpy.zeros((n_batch,), dtype="float32")
        err = numpy.zeros(log_posteriors.shape, dtype="float32")
        queue = sorted(range(n_batch), key=lambda b: -int(seq_lengths[b]))  # longest first
        running: Dict[int, int] = {}  # fileno -> batch index

        def feed(inst: SprintSubprocessInstance) -> bool:
            if not queue:
                return False
            b = queue.pop(0)
            n = int(seq_lengths[b])
            inst.get_loss_and_error_signal__send(seg_name=tags[b], seg_len=n, log_posteriors=log_posteriors[:n, b])
            running[inst.fileno()] = b
            return True

        with selectors.DefaultSelector() as sel:
            for i in range(min(self.max_num_instances, n_batch)):
                inst = self._get_instance(i)
                feed(inst)
                sel.register(inst.fileno(), selectors.EVENT_READ, inst)
            while running:
                for key, _ in sel.select():
                    inst = key.data
                    b = running.pop(inst.fileno())
                    name, loss_b, err_b = inst.get_loss_and_error_signal__read()
                    assert name == tags[b]
                    loss[b] = loss_b
                    err[: int(seq_lengths[b]), b] = err_b
                    feed(inst)
        return loss, err

    def get_automata_for_batch(self, tags: Sequence[str]) -> Tuple[numpy.ndarray, numpy.ndarray, numpy.ndarray]:
        """
        :return: edges [4, E] uint32 as rows (from, to, emission, sequence index) with state numbers offset so that all sequences share one
            state space; weights [E] float32; start_end_states [2, B] uint32
        """
        parts = []
        for bb in range(0, len(tags), self.max_num_instances):
            chunk = list(range(bb, min(bb + self.max_num_instances, len(tags))))
            for i, b in enumerate(chunk):
                tag = tags[b].decode("utf8") if isinstance(tags[b], bytes) else str(tags[b])
                self._get_instance(i)._send(("export_allophone_state_fsa_by_segment_name", tag))
            for i, b in enumerate(chunk):
                ret = self._get_instance(i)._read()
                if ret[0] != "ok":
                    raise RuntimeError("RASR child failed on the automaton of %r: %s" % (tags[b], ret[1:]))
                parts.append(ret[1:])
        edges, weights, offset = [], [], 0
        start_end = numpy.empty((2, len(tags)), dtype="uint32")
        for b, (num_states, num_edges, e, w) in enumerate(parts):
            e = numpy.array(e, dtype="uint32").reshape(3, num_edges)
            e[0:2] += offset
            edges.append(numpy.vstack([e, numpy.full((1, num_edges), b, dtype="uint32")]))
            weights.append(numpy.asarray(w, dtype="float32"))
            start_end[:, b] = (offset, offset + num_states - 1)
            offset += num_states
        return numpy.hstack(edges), numpy.hstack(weights), start_end


def sprint_loss(log_probs, seq_lens, tags: Sequence[str], sprint_opts: Dict[str, Any]):
    """
    :param torch.Tensor log_probs: [B, T, D] log posteriors (any device)
    :param seq_lens: [B] lengths (tensor or array)
    :param tags: B sequence names
    :param sprint_opts: options of :class:`SprintInstancePool`
    :return: [B] losses; the gradient w.r.t. ``log_probs`` is RASR's error signal, scaled by the incoming gradient per sequence
    """
    import torch

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            pool = SprintInstancePool.get_global_instance(sprint_opts)
            lens = numpy.asarray(seq_lens.detach().cpu() if isinstance(seq_lens, torch.Tensor) else seq_lens, dtype="int32")
            x_tbd = x.detach().float().transpose(0, 1).contiguous().cpu().numpy()
            with pool.lock:
                loss, err = pool.get_batch_loss_and_error_signal(x_tbd, lens, list(tags))
            ctx.save_for_backward(torch.from_numpy(err).transpose(0, 1).to(device=x.device, dtype=x.dtype))
            return torch.from_numpy(loss).to(x.device)

        @staticmethod
        def backward(ctx, grad_loss):
            (err,) = ctx.saved_tensors
            return err * grad_loss.to(err.dtype)[:, None, None]

    return _Fn.apply(log_probs)
