"""
The module a RASR ("Sprint") process loads to serve a trainer in ANOTHER process: the trainer (see ``error_signals.py``) starts
RASR as a child with ``--*.pymod-name=returnn_b200.sprint.control`` and two pipe descriptors in ``--*.pymod-config``; RASR imports this
module, calls :func:`init` and then hands its thread to :meth:`PythonControl.run_control_loop`. From then on the trainer sends
commands over the pipe and RASR's own code answers them through the callback it gave to the loop:

=============================================  ======================================================================
command from the trainer                       answer
=============================================  ======================================================================
``("init", name, version)``                    ``("ok", "SprintControl", version)``
``("get_loss_and_error_signal", seg, T, x)``   ``("ok", loss, error_signal[T, D])``; x are (log) posteriors [T, D]
``("export_allophone_state_fsa_by_segment_name", seg)``  ``("ok", num_states, num_edges, edges, weights)``
``("exit",)``                                  none; the pipes close and the loop ends with ``SystemExit``
=============================================  ======================================================================

A failing command answers ``("exception", message)`` and the loop goes on. Messages are length-prefixed pickles
(``utils.basic.write_pickled_object``).

With ``--*.python-segment-order=true`` RASR also asks :func:`getSegmentList` for its segment order: the iterator yields the segment of
each ``get_loss_and_error_signal`` command as it arrives, so RASR processes exactly the sequences the trainer's batches hold, in
their order. In that mode the control loop runs in a thread of its own and the criterion comes from RASR's trainer calling
:meth:`PythonControl.get_current_seg_posteriors` / :meth:`PythonControl.set_current_seg_error_signal` around its own computation.

Parity: returnn/sprint/control.py (``init`` :55, ``getSegmentList`` :128, ``SprintNnPythonLayer`` :152, ``PythonControl`` :278).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional
import os
import sys
import threading
import numpy

from ..utils.basic import read_pickled_object, write_pickled_object

Verbose = False
Quiet = False
InitTypes = set()


def _log(*args):
    if not Quiet:
        print("returnn_b200 SprintControl[pid %i]" % os.getpid(), *args, file=sys.stderr, flush=True)


def _parse_config(config: str) -> Dict[str, str]:
    return dict(item.split(":", 1) for item in config.split(",") if item)


def _to_bool(v) -> bool:
    return str(v).lower() in ("1", "true", "yes", "y", "on")


def init(name, reference, config, sprint_unit=None, version_number=None, callback=None, **kwargs):
    """
    Called by RASR's PythonControl (and by :func:`getSegmentList` / :class:`SprintNnPythonLayer` here).

    :param str name: who calls, e.g. "Sprint.PythonControl"
    :param reference: any object identifying the caller's instance
    :param str config: ``key:value,...`` from ``--*.pymod-config``; needs ``c2p_fd``, ``p2c_fd``, ``minPythonControlVersion``
    :param sprint_unit: which part of RASR, e.g. "NnTrainer.pythonControl"
    :param version_number: of RASR's PythonControl
    :param callback: ``callback(action, **args)`` into RASR
    :return: the :class:`PythonControl` singleton
    """
    global Verbose, Quiet
    opts = _parse_config(config)
    Quiet = Quiet or _to_bool(opts.get("quiet", False))
    Verbose = Verbose or _to_bool(opts.get("verbose", False))
    InitTypes.add(name)
    _log("init: name=%r sprint_unit=%r version_number=%r" % (name, sprint_unit, version_number))
    return PythonControl.create(c2p_fd=int(opts["c2p_fd"]), p2c_fd=int(opts["p2c_fd"]), name=name, reference=reference, config=opts, sprint_unit=sprint_unit,
                                version_number=version_number, min_version_number=int(opts.get("minPythonControlVersion", 0)), callback=callback, **kwargs)


def getSegmentList(corpusName, segmentList, config, **_kwargs):
    """RASR's PythonSegmentOrder: yields the segment names the trainer asks for, one per command"""
    init(name="RETURNN.PythonSegmentOrder", reference=corpusName, config=config)
    PythonControl.instance.check_control_loop_running()
    for name in PythonControl.instance.segment_list_iterator():
        yield name.decode("utf8") if isinstance(name, bytes) else name


class SprintNnPythonLayer:
    """
    RASR's ``NnPythonLayer``: a network layer whose forward output are the trainer's posteriors for the current segment and whose
    backward input is RASR's error signal for them (which goes back to the trainer).
    """

    def __init__(self, config, **kwargs):
        init(name="RETURNN.SprintNnPythonLayer", reference=self, config=config)
        self.input_size = None
        self.output_size = None

    def finalize(self):
        """RASR is done with the layer"""

    def setInputDimension(self, stream, size):
        """:param int stream: only one input stream is used"""
        assert stream == 0
        self.input_size = size

    def setOutputDimension(self, size):
        """number of classes"""
        self.output_size = size

    def initializeNetworkParameters(self):
        """no parameters live on this side"""

    def loadNetworkParameters(self, filename):
        """no parameters live on this side"""

    def saveNetworkParameters(self, filename):
        """no parameters live on this side"""

    def isTrainable(self):
        """so that RASR calls :meth:`backpropagate`"""
        return True

    def getNumberOfFreeParameters(self):
        """none on this side"""
        return 0

    def forward(self, input):
        """:param input: tuple of (input_size, T) arrays; :return: (output_size, T) posteriors of the trainer"""
        assert len(input) == 1
        n_time = input[0].shape[1]
        seg_len = PythonControl.instance.get_current_seg_posteriors(n_time)  # (T, D)
        assert seg_len.shape == (n_time, self.output_size)
        return seg_len.T

    def backpropagate(self, errorSignalIn):
        """:param errorSignalIn: (output_size, T); :return: tuple with a zero error signal for the (unused) input"""
        assert errorSignalIn.shape[0] == self.output_size
        n_time = errorSignalIn.shape[1]
        PythonControl.instance.set_current_seg_error_signal(n_time, errorSignalIn.T)
        return (numpy.zeros((self.input_size, n_time), dtype="float32"),)


class PythonControl:
    """the object RASR talks to; one per process"""

    Version = 1  # of the pipe protocol; the trainer checks it
    instance: Optional["PythonControl"] = None

    @classmethod
    def create(cls, **kwargs) -> "PythonControl":
        """the singleton; later calls only repeat the per-caller part of the initialisation"""
        if cls.instance is None:
            cls.instance = cls(**kwargs)
        else:
            cls.instance._init(**kwargs)
        return cls.instance

    def __init__(self, c2p_fd: int, p2c_fd: int, **kwargs):
        self.cond = threading.Condition()
        self.pipe_c2p = os.fdopen(c2p_fd, "wb")
        self.pipe_p2c = os.fdopen(p2c_fd, "rb")
        self.sprint_callback: Optional[Callable] = None
        self.callback: Optional[Callable] = None
        self.sprint_version_number = None
        self.control_loop_started = False
        self.control_loop_exited = False
        self.control_thread: Optional[threading.Thread] = None
        self.control_thread__have_new_seg = False
        self.control_thread__have_new_error_signal = False
        self.seg_name: Optional[str] = None
        self.seg_len: Optional[int] = None
        self.posteriors: Optional[numpy.ndarray] = None
        self.asked_for_posteriors = False
        self.notified_for_segment = False
        self.error_signal: Optional[numpy.ndarray] = None
        self.loss: Optional[float] = None
        self.posteriors_in_log_space = True
        self.sprint_knows_about_log_space_probs = False
        self._init(**kwargs)

    def _init(self, name=None, sprint_unit=None, callback=None, version_number=None, min_version_number=None, config=None, **_kwargs):
        if name == "Sprint.PythonControl":
            self.sprint_callback = callback
            self.sprint_version_number = version_number
            if min_version_number:
                assert (version_number or 0) >= min_version_number, "RASR's PythonControl is version %r, needed is %r" % (version_number, min_version_number)
        if config:
            self.posteriors_in_log_space = _to_bool(config.get("posteriors_in_log_space", self.posteriors_in_log_space))
            self.sprint_knows_about_log_space_probs = _to_bool(config.get("sprint_knows_about_log_space_probs", self.sprint_knows_about_log_space_probs))

    # -- calls from RASR --

    def init_processing(self, input_dim=None, output_dim=None, **_kwargs):
        """before the first segment of a corpus pass"""
        _log("init_processing: input_dim=%r output_dim=%r" % (input_dim, output_dim))

    def process_segment(self, name, orthography, features=None, alignment=None, soft_alignment=None, **_kwargs):
        """
        RASR iterates its corpus itself (``extract-features`` style) and hands over one segment: the posteriors come from the trainer,
        the criterion from RASR's ``calculate_criterion`` callback, the result goes back to the trainer.
        """
        assert self.sprint_callback is not None, "RASR's PythonControl gave no callback"
        seg_len = features.shape[1] if features is not None else None
        posteriors = self.get_current_seg_posteriors(seg_len)
        loss, err = self._criterion_via_sprint_callback(name, orthography, posteriors)
        self.set_current_seg_loss(name, loss)
        self.set_current_seg_error_signal(posteriors.shape[0], err)

    def _criterion_via_sprint_callback(self, seg_name, orthography, posteriors: numpy.ndarray):
        if self.posteriors_in_log_space and self.sprint_knows_about_log_space_probs:
            kind = "error-signal"  # RASR returns the gradient w.r.t. the activations before the softmax
        else:
            kind = "error-signal-before-softmax"
            if self.posteriors_in_log_space:
                posteriors = numpy.exp(posteriors)
        loss, err = self.sprint_callback("calculate_criterion", posteriors=posteriors.T, orthography=orthography, output_error_type=kind,
                                         segment_name=seg_name)  # RASR works on (D, T)
        if loss is None:  # RASR skipped the segment (no path through the lattice, ...)
            return 0.0, numpy.zeros_like(posteriors, dtype="float32")
        err = err.T
        assert err.shape == posteriors.shape
        return loss, err

    def exit(self, **kwargs):
        """RASR ends"""
        _log("exit: %r" % (kwargs,))

    def run_control_loop(self, callback, **kwargs):
        """RASR gives its thread away: read commands until ``exit``"""
        self.callback = callback
        with self.cond:
            assert not self.control_loop_started
            self.control_loop_started = True
            self.cond.notify_all()
        try:
            while True:
                self.handle_next()
        finally:
            with self.cond:
                self.control_loop_exited = True
                self.cond.notify_all()

    # -- the pipe --

    def _send(self, data):
        write_pickled_object(self.pipe_c2p, data)

    def _read(self):
        return read_pickled_object(self.pipe_p2c)

    def close(self):
        """both pipe ends"""
        self.pipe_c2p.close()
        self.pipe_p2c.close()

    def handle_next(self):
        """one command: read, dispatch to ``_handle_cmd_<name>``, answer"""
        args = self._read()
        try:
            assert isinstance(args, tuple) and args, "a command is a tuple (name, ...), got %r" % (args,)
            res = getattr(self, "_handle_cmd_%s" % args[0])(*args[1:])
        except Exception as exc:
            import traceback

            _log("command %r failed:\n%s" % (args[0] if isinstance(args, tuple) and args else args, traceback.format_exc()))
            self._send(("exception", "%s: %s" % (type(exc).__name__, exc)))
        else:
            assert isinstance(res, tuple)
            self._send(("ok",) + res)

    def _handle_cmd_exit(self):
        self.close()
        raise SystemExit

    def _handle_cmd_init(self, name, version):
        assert version == self.Version, "trainer speaks protocol version %r, this module %r" % (version, self.Version)
        return "SprintControl", self.Version

    def _handle_cmd_get_loss_and_error_signal(self, seg_name, seg_len, posteriors):
        seg_len = int(seg_len)
        assert seg_len > 0 and posteriors.ndim == 2 and posteriors.shape[0] == seg_len
        with self.cond:
            self.control_thread__have_new_seg = True
            self.control_thread__have_new_error_signal = False
            self.seg_name = seg_name.decode("utf8") if isinstance(seg_name, bytes) else seg_name
            self.seg_len = seg_len
            self.posteriors = posteriors
            self.error_signal = self.loss = None
            self.asked_for_posteriors = self.notified_for_segment = False
            self.cond.notify_all()
        loss, err = self.callback("get_loss_and_error_signal", seg_name, seg_len, posteriors)
        assert err.shape == posteriors.shape
        with self.cond:
            self.control_thread__have_new_error_signal = True
            self.posteriors = None
            self.cond.notify_all()
        return float(loss), numpy.ascontiguousarray(err, dtype="float32")

    def _handle_cmd_export_allophone_state_fsa_by_segment_name(self, segment_name):
        return tuple(self.callback("export_allophone_state_fsa_by_segment_name", segment_name))

    # -- RASR as the driver (segment order + NnPythonLayer): the loop runs in a thread of this module --

    def check_control_loop_running(self):
        """start the threaded loop unless RASR runs it"""
        if not self.control_loop_started:
            self.run_threaded_control_loop()

    def run_threaded_control_loop(self):
        """the command loop in a daemon thread; the criterion then comes from RASR's trainer thread through the ``own_tcb_*`` calls"""
        def loop():
            try:
                self.run_control_loop(self.own_threaded_callback)
            except SystemExit:
                pass
            except BaseException:
                sys.excepthook(*sys.exc_info())
                os._exit(1)  # the trainer waits on the pipe: end the process rather than leave it waiting

        self.control_thread = threading.Thread(target=loop, name="SprintControl.PythonControl.threaded_control_loop", daemon=True)
        self.control_thread.start()

    def own_threaded_callback(self, cmd, *args):
        """stands in for RASR's callback when the loop is threaded"""
        return getattr(self, "own_tcb_%s" % cmd)(*args)

    def own_tcb_version(self):
        """:return: a version string for the log"""
        return "<version>returnn_b200.sprint.control.PythonControl.threaded</version>"

    def own_tcb_get_loss_and_error_signal(self, seg_name, seg_len, posteriors):
        """waits until RASR's trainer thread has delivered the error signal of this segment"""
        with self.cond:
            while self.error_signal is None or self.loss is None:
                assert not self.control_loop_exited
                self.cond.wait(1.0)
            return self.loss, self.error_signal

    def init_segment(self, segment_name):
        """RASR's trainer announces the segment it works on"""
        with self.cond:
            assert self.seg_name == segment_name, "RASR works on %r, the trainer asked for %r" % (segment_name, self.seg_name)
            self.notified_for_segment = True
            self.cond.notify_all()

    def notify_segment_loss(self, segment_name, loss):
        """RASR's trainer reports the loss"""
        self.set_current_seg_loss(segment_name, loss)

    def get_current_seg_posteriors(self, seg_len):
        """:return: [T, D] posteriors of the segment the trainer sent last"""
        with self.cond:
            assert self.control_loop_started and self.posteriors is not None
            if seg_len is not None:
                assert self.seg_len == seg_len, "segment %r: RASR has %r frames, the trainer %r" % (self.seg_name, seg_len, self.seg_len)
            self.asked_for_posteriors = True
            self.cond.notify_all()
            return self.posteriors

    def set_current_seg_error_signal(self, seg_len, error_signal):
        """:param error_signal: [T, D]"""
        with self.cond:
            assert self.seg_len == seg_len and error_signal.ndim == 2 and error_signal.shape[0] == seg_len
            self.error_signal = error_signal
            self.cond.notify_all()

    def set_current_seg_loss(self, seg_name, loss):
        """:param seg_name: may be None when RASR does not say"""
        with self.cond:
            if seg_name:
                assert self.seg_name == seg_name
            self.loss = loss
            self.cond.notify_all()

    def _skip_segment_loss_and_error(self):
        with self.cond:
            assert self.posteriors is not None
            if self.loss is None:
                self.loss = 0.0
            if self.error_signal is None:
                self.error_signal = numpy.zeros_like(self.posteriors, dtype="float32")
            self.cond.notify_all()

    def _wait_for_control_loop_error_signal(self):
        """after yielding a segment: RASR must have asked for its posteriors and delivered the signal, else the segment was skipped"""
        with self.cond:
            while not self.control_thread__have_new_error_signal and not self.control_loop_exited:
                if self.error_signal is None and self.posteriors is not None and not self.asked_for_posteriors and not self.notified_for_segment:
                    # RASR came back for the next segment without touching this one
                    self._skip_segment_loss_and_error()
                self.cond.wait(1.0)

    def segment_list_iterator(self):
        """yields each segment the trainer asks for; ends when the trainer sends ``exit``"""
        with self.cond:
            while True:
                while not self.control_thread__have_new_seg and not self.control_loop_exited:
                    self.cond.wait(1.0)
                if self.control_loop_exited:
                    return
                self.control_thread__have_new_seg = False
                name = self.seg_name
                self.cond.release()
                try:
                    yield name
                finally:
                    self.cond.acquire()
                self._wait_for_control_loop_error_signal()
