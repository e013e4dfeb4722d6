"""
This framework INSIDE a RASR ("Sprint") process: RASR loads this module (``--*.pymod-name=returnn_b200.sprint.interface``) as its
PythonTrainer, PythonSegmentOrder and/or PythonFeatureScorer and calls the functions below.

* trainer, ``action:train``: RASR extracts features (and alignments) and feeds them sequence by sequence (``feedInputAndTarget*``);
  they land in a :class:`~returnn_b200.datasets.sprint.SprintDatasetBase`, and the engine trains from that dataset in a thread of
  its own. With the segment order taken from :func:`getSegmentList`, RASR walks the corpus once per epoch in the order the dataset's
  ``seq_ordering`` asks for.
* trainer, ``action:forward``: every fed sequence runs through the model's forward step; the posteriors go back to RASR as ``[D, T]``.
* feature scorer: RASR's decoder adds frames (``add_feature``), asks for a block to be computed (``compute``) and reads scores
  ``-log p(class | x) + prior_scale * log prior(class)`` per frame (``get_scores``).

All state sits in one :class:`_Session` object (``session``); the module-level functions are the names RASR looks up.

Parity: returnn/sprint/interface.py (``init`` :65, ``PythonFeatureScorer`` :132, ``getSegmentList`` :332, ``init_python_trainer``
:407, ``exit`` :477, ``feedInput*`` :502-648, ``_init_base`` :700, ``_start_train_thread`` :775, ``_forward`` :935).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional
import os
import sys
import threading
import time
import numpy

DefaultSprintCrnnConfig = "config/crnn.config"


def _parse_config(config: str) -> Dict[str, str]:
    return dict(item.split(":", 1) for item in (config or "").split(",") if item)


class _Session:
    """everything the calls below share"""

    def __init__(self):
        self.config = None
        self.engine = None
        self.sprint_dataset = None
        self.custom_dataset = None
        self.task: Optional[str] = None  # "train", "forward", "nop"
        self.target_mode: Optional[str] = None
        self.input_dim: Optional[int] = None
        self.output_dim: Optional[int] = None
        self.max_segment_length = 1
        self.train_thread: Optional[threading.Thread] = None
        self.train_error: Optional[BaseException] = None
        self.start_time: Optional[float] = None
        self.initialized = False
        self.exited = False

    # -- set-up --

    def init_base(self, configfile: Optional[str] = None, target_mode: Optional[str] = None, epoch: Optional[int] = None,
                  sprint_opts: Optional[Dict[str, str]] = None):
        """config, log, dataset, engine: each only once, so that segment order and trainer may both call this"""
        from .. import __main__ as rnn

        self.initialized = True
        if not getattr(sys, "argv", None):
            sys.argv = [__file__]  # an embedded interpreter has none
        if self.config is None:
            configfile = configfile or DefaultSprintCrnnConfig
            assert os.path.exists(configfile), "config file %r not found" % configfile
            rnn.init_config(config_filename=configfile, extra_updates={"task": target_mode or "train"})
            self.config = rnn.config
            for key, value in (sprint_opts or {}).items():
                if key not in ("action", "configfile", "epoch"):
                    self.config.set(key, value)
            rnn.init_log()
            rnn.returnn_greeting(config_filename=configfile)
            rnn.init_backend_engine()
            rnn.init_faulthandler(sigusr1_chain=True)
        if target_mode:
            self.set_target_mode(target_mode)
        self.init_dataset()
        if target_mode == "forward" and epoch:
            from ..engine.base import EngineBase

            model = self.config.value("model", "")
            found = [fn for fn in (EngineBase.epoch_model_filename(model, epoch, is_pretrain=p) for p in (False, True)) if os.path.exists(fn + ".pt")]
            assert len(found) == 1, "no checkpoint of epoch %i for model %r" % (epoch, model)
            self.config.set("load", found[0])
        if self.engine is None:
            rnn.print_task_properties()
            rnn.init_engine()
            self.engine = rnn.engine

    def init_dataset(self):
        """the dataset RASR feeds (options from ``sprint_interface_dataset_opts``); optionally a user dataset wrapped around it"""
        if self.sprint_dataset is not None:
            return
        from ..datasets.sprint import SprintDatasetBase
        from ..datasets.basic import init_dataset

        opts = dict(self.config.typed_value("sprint_interface_dataset_opts", None) or {})
        if "seq_ordering" not in opts and self.config.value("batching", None):
            opts["seq_ordering"] = self.config.value("batching", None)  # the config key of the order for the main training data
        self.sprint_dataset = SprintDatasetBase(**opts)
        make_custom = self.config.typed_value("sprint_interface_custom_dataset", None)
        if callable(make_custom):
            self.custom_dataset = init_dataset(make_custom(sprint_dataset=self.sprint_dataset))

    def set_target_mode(self, mode: str):
        """
        :param mode: "target-alignment" (frame labels from RASR), "criterion-by-sprint" (RASR computes the criterion), "forward"
        """
        assert self.config is not None
        self.target_mode = mode
        task = {"criterion-by-sprint": "train", "target-alignment": "train", "forward": "forward"}.get(mode)
        assert task, "target mode %r" % mode
        self.config.set("task", task)
        if mode == "forward":
            self.config.set("extract", "posteriors")

    def get_final_epoch(self) -> int:
        """last epoch of the training"""
        from ..engine.base import EngineBase

        return EngineBase.config_get_final_epoch(self.config)

    def get_start_epoch(self) -> int:
        """first epoch (after the newest checkpoint)"""
        from ..engine.base import EngineBase

        return EngineBase.get_train_start_epoch(self.config)

    # -- training --

    def start_train_thread(self, epoch: Optional[int] = None):
        """the engine trains from the fed dataset while RASR's thread keeps feeding"""
        assert self.initialized and self.train_thread is None and self.sprint_dataset is not None and self.task == "train"
        assert self.target_mode == "target-alignment", "target mode %r is not supported for training inside RASR" % self.target_mode

        def run():
            try:
                self.engine.init_train_from_config(self.config, train_data=self.custom_dataset or self.sprint_dataset)
                if epoch is not None:
                    assert epoch == self.engine.start_epoch, "RASR asks for epoch %i, the checkpoints continue at %i" % (epoch, self.engine.start_epoch)
                self.engine.train()
            except KeyboardInterrupt:
                pass
            except BaseException as exc:  # RASR's thread must not go on feeding a trainer that is gone
                self.train_error = exc
                sys.excepthook(*sys.exc_info())
                import _thread

                _thread.interrupt_main()

        self.train_thread = threading.Thread(target=run, name="RASR-fed train thread", daemon=True)
        self.train_thread.start()

    def train_seq(self, segment_name: Optional[str], features: numpy.ndarray, targets=None):
        """:param features: [D, T] as RASR gives them"""
        assert self.train_thread is not None, "not initialised as a trainer"
        if self.train_error is not None:
            raise RuntimeError("the train thread failed") from self.train_error
        assert features.shape[0] == self.input_dim
        if targets is None:
            assert self.target_mode != "target-alignment"
        self.sprint_dataset.add_new_data(features, targets, segment_name=segment_name)

    # -- forwarding --

    def prepare_forwarding(self):
        """load the model"""
        self.engine.init_network_from_config(self.config)

    def features_to_dataset(self, features: numpy.ndarray, segment_name: Optional[str]):
        """:param features: [D, T]; :return: a one-sequence dataset"""
        from ..datasets.generating import StaticDataset

        assert features.shape[0] == self.input_dim
        ds = StaticDataset(data=[{"data": numpy.ascontiguousarray(features.T, dtype="float32"), "seq_tag": segment_name or "seq-0"}], target_list=[],
                           output_dim={"data": (self.input_dim, 2)})
        ds.init_seq_order(epoch=1)
        return ds

    def forward(self, segment_name: Optional[str], features: numpy.ndarray) -> numpy.ndarray:
        """:param features: [D_in, T]; :return: posteriors [D_out, T]"""
        from ..forward_iface import ForwardCallbackIface

        got: List[numpy.ndarray] = []

        class _Collect(ForwardCallbackIface):
            def process_seq(self, *, seq_tag, outputs):
                out = outputs["output"] if "output" in outputs.data else next(iter(outputs.data.values()))
                got.append(numpy.asarray(out.raw_tensor))

        ds = self.features_to_dataset(features, segment_name)
        self.engine.forward_with_callback(dataset=ds, callback=_Collect(), dataset_init_epoch=False)
        assert len(got) == 1
        post = got[0]
        assert post.ndim == 2 and post.shape[0] == features.shape[1], "the model output must keep one frame per input frame"
        if self.output_dim:
            assert post.shape[1] == self.output_dim, "model output has %i classes, RASR expects %i" % (post.shape[1], self.output_dim)
        return numpy.ascontiguousarray(post.T, dtype="float32")

    # -- end --

    def exit(self):
        """join the train thread (RASR has fed everything)"""
        if self.exited:
            return
        self.exited = True
        if self.train_thread is not None:
            self.sprint_dataset.finalize_sprint()
            self.train_thread.join()
            self.train_thread = None
            if self.train_error is not None:
                raise RuntimeError("the train thread failed") from self.train_error
        if self.start_time is not None:
            print("SprintInterface[pid %i]: elapsed %.1f s" % (os.getpid(), time.time() - self.start_time), file=sys.stderr)


session = _Session()


# ---- entry points RASR calls (their names and argument names are RASR's) ----


def init(name=None, sprint_unit=None, **kwargs):
    """first call of every RASR component that loads this module"""
    print("SprintInterface[pid %i] init: name=%r sprint_unit=%r" % (os.getpid(), name, sprint_unit), file=sys.stderr)
    if name is None or sprint_unit == "PythonFeatureScorer":  # older RASR versions give no name to the trainer
        if sprint_unit == "PythonFeatureScorer":
            return init_python_feature_scorer(**kwargs)
        return init_python_trainer(**kwargs)
    if name == "Sprint.PythonControl" and sprint_unit in ("FeedForwardTrainer", "SegmentwiseNnTrainer", "NnTrainer.pythonControl", None):
        return None  # nothing to control from here: the trainer interface below is used
    raise Exception("SprintInterface: unknown caller name=%r sprint_unit=%r" % (name, sprint_unit))


def init_python_feature_scorer(config, **kwargs):
    """:return: the :class:`PythonFeatureScorer` RASR's decoder talks to"""
    opts = _parse_config(config)
    epoch = int(opts["epoch"]) if opts.get("epoch") else None
    session.task = "forward"
    session.init_base(target_mode="forward", configfile=opts.get("configfile"), epoch=epoch, sprint_opts=opts)
    return PythonFeatureScorer(sprint_opts=opts, **kwargs)


class PythonFeatureScorer:
    """acoustic scores for RASR's decoder"""

    def __init__(self, sprint_opts: Dict[str, str], callback=None, version_number=None, **_kwargs):
        self.sprint_opts = sprint_opts
        self.callback = callback
        self.version_number = version_number
        self.input_dim = self.output_dim = None
        self.priors: Optional[numpy.ndarray] = None
        self.prior_scale = float(sprint_opts.get("prior_scale", session.config.float("prior_scale", 1.0) if session.config else 1.0))
        self.segment_count = 0
        self.features: List[numpy.ndarray] = []
        self.scores: Optional[numpy.ndarray] = None

    def init(self, input_dim, output_dim):
        """dimensions of RASR's features and label set"""
        self.input_dim, self.output_dim = input_dim, output_dim
        session.input_dim, session.output_dim = input_dim, output_dim
        session.sprint_dataset.set_dimensions(input_dim, output_dim)
        session.prepare_forwarding()
        self._load_priors()

    def _load_priors(self):
        fn = self.sprint_opts.get("prior_file") or (session.config.value("prior_file", None) if session.config else None)
        if not fn:
            return
        pri = numpy.loadtxt(fn, dtype="float32").reshape(-1)
        assert pri.shape == (self.output_dim,), "prior file %r has %i entries, expected %i" % (fn, pri.size, self.output_dim)
        if pri.max() > 0 or abs(numpy.exp(pri).sum() - 1.0) > 0.1:  # probabilities, not log probabilities
            pri = numpy.log(numpy.maximum(pri, 1e-30))
        self.priors = pri

    def exit(self):
        """decoder is done"""
        session.exit()

    def get_feature_buffer_size(self) -> int:
        """-1: whole segments are buffered before :meth:`compute`"""
        return -1

    def add_feature(self, feature, time):
        """:param feature: [D]; :param time: frame index within the segment"""
        assert time == len(self.features) and feature.shape == (self.input_dim,)
        self.features.append(numpy.array(feature, dtype="float32"))

    def reset(self, num_frames):
        """a segment ends"""
        assert num_frames == len(self.features)
        self.features = []
        self.scores = None
        self.segment_count += 1

    def get_segment_name(self) -> str:
        """RASR does not say which segment it decodes"""
        return "unknown-seq-name-%i" % self.segment_count

    def get_features(self, num_frames=None) -> numpy.ndarray:
        """:return: [D, T]"""
        if num_frames is not None:
            assert num_frames == len(self.features)
        return numpy.stack(self.features, axis=1)

    def get_posteriors(self, num_frames=None) -> numpy.ndarray:
        """:return: [D_out, T]"""
        post = session.forward(self.get_segment_name(), self.get_features(num_frames))
        assert post.shape == (self.output_dim, len(self.features))
        return post

    def compute(self, num_frames):
        """scores of all buffered frames"""
        post = self.get_posteriors(num_frames)
        scores = -numpy.log(numpy.maximum(post, 1e-30))
        if self.priors is not None:
            scores = scores + self.prior_scale * self.priors[:, None]
        self.scores = scores

    def get_scores(self, time) -> numpy.ndarray:
        """:return: [D_out] scores (negative log, prior divided out) of frame ``time``"""
        assert self.scores is not None, "compute() first"
        return self.scores[:, time]


def getSegmentList(corpusName, segmentList, **kwargs):
    """
    RASR's PythonSegmentOrder: all segments once per epoch in the dataset's order, from the start epoch to the last; RASR thereby
    walks as many passes over the corpus as there are epochs left.
    """
    session.init_base(configfile=kwargs.get("config"))
    ds = session.sprint_dataset
    ds.use_multiple_epochs()
    start, final = session.get_start_epoch(), session.get_final_epoch()
    print("SprintInterface: %i segments in %r, epochs %i..%i" % (len(segmentList), corpusName, start, final), file=sys.stderr)
    for epoch in range(start, final + 1):
        if session.train_thread is not None:
            ds.wait_for_returnn_epoch(epoch)  # the trainer has closed the previous epoch before its window is reset
        ds.init_sprint_epoch(epoch)
        order = ds.get_seq_order_for_epoch(epoch, len(segmentList))
        for i, idx in enumerate(order):
            ds.set_complete_frac(float(i + 1) / len(order))
            yield segmentList[idx]
        ds.finish_sprint_epoch()
        if session.train_thread is not None:
            assert ds.get_num_timesteps() > 0, "no sequence arrived in epoch %i: is RASR's feature buffer larger than the corpus?" % epoch
    ds.finalize_sprint()


def init_python_trainer(inputDim, outputDim, config, targetMode, **kwargs):
    """RASR's PythonTrainer (``trainer = python-trainer``); called late, with the first data"""
    session.input_dim, session.output_dim = inputDim, outputDim
    session.max_segment_length = kwargs.get("maxSegmentLength", session.max_segment_length)
    opts = _parse_config(config)
    epoch = int(opts["epoch"]) if opts.get("epoch") else None
    assert epoch is None or epoch >= 1
    action = opts["action"]
    assert action in ("train", "forward", "nop"), "unknown action %r" % action
    session.task = action
    if action == "forward":
        assert targetMode in ("criterion-by-sprint", "forward-only")
        targetMode = "forward"
    elif action == "nop":
        targetMode = None
    session.init_base(target_mode=targetMode, configfile=opts.get("configfile"), epoch=epoch, sprint_opts=opts)
    session.sprint_dataset.set_dimensions(inputDim, outputDim)
    session.sprint_dataset.initialize()
    if action == "train":
        session.start_train_thread(epoch)
    elif action == "forward":
        session.prepare_forwarding()
    session.start_time = time.time()


def exit():
    """RASR ends"""
    session.exit()


def feedInput(features, weights=None, segmentName=None):
    """:param features: [D, T]; :return: posteriors [D_out, T] when forwarding"""
    if session.task == "train":
        session.train_seq(segmentName, features)
        return None
    if session.task == "forward":
        return session.forward(segmentName, features)
    raise Exception("feedInput: task %r" % session.task)


def finishDiscard():
    """RASR drops the criterion result of the last segment"""
    raise NotImplementedError("criterion-by-sprint inside RASR is not supported: use sprint.error_signals from the trainer's side")


def finishError(error, errorSignal, naturalPairingType=None):
    """RASR's criterion result for the last segment"""
    raise NotImplementedError("criterion-by-sprint inside RASR is not supported: use sprint.error_signals from the trainer's side")


def feedInputAndTarget(features, weights=None, segmentName=None, orthography=None, alignment=None, speaker_name=None, speaker_gender=None, **kwargs):
    """newer RASR versions: everything by keyword"""
    targets: Dict[str, Any] = {}
    if alignment is not None:
        targets["classes"] = alignment
    if orthography is not None:
        targets["orth"] = orthography
    if speaker_name is not None:
        targets["speaker_name"] = speaker_name
    if speaker_gender is not None:
        targets["speaker_gender"] = speaker_gender
    session.train_seq(segmentName, features, targets)


def feedInputAndTargetAlignment(features, targetAlignment, weights=None, segmentName=None):
    """:param targetAlignment: [T] class indices"""
    session.train_seq(segmentName, features, {"classes": targetAlignment})


def feedInputAndTargetSegmentOrth(features, targetSegmentOrth, weights=None, segmentName=None):
    """:param targetSegmentOrth: transcription"""
    session.train_seq(segmentName, features, {"orth": targetSegmentOrth})


def feedInputUnsupervised(features, weights=None, segmentName=None):
    """no targets"""
    session.train_seq(segmentName, features)


def feedInputForwarding(features, weights=None, segmentName=None):
    """:return: posteriors [D_out, T]"""
    assert session.task == "forward"
    return session.forward(segmentName, features)


def dump_flags():
    """for RASR's log"""
    print("SprintInterface flags: task=%r target_mode=%r input_dim=%r output_dim=%r" % (session.task, session.target_mode, session.input_dim, session.output_dim),
          file=sys.stderr)


def set_target_mode(mode):
    """see :meth:`_Session.set_target_mode`"""
    session.set_target_mode(mode)
