"""
Python module loaded by RASR (``--*.pymod-name=returnn_b200.sprint.extern_interface``) when it is started by
:class:`returnn_b200.datasets.sprint.ExternSprintDataset`. RASR calls the entry points below by their fixed names:
``getSegmentList`` (its PythonSegmentOrder hook), and ``init`` / ``feedInput*`` / ``exit`` (PythonTrainer) or the
``PythonControl`` class (``--*.python-control-enabled``). Everything that arrives is forwarded as length-prefixed pickled
messages over the pipe whose descriptor the parent put into ``pymod-config`` (``c2p_fd``).

Parity: returnn/sprint/extern_interface.py (getSegmentList :25, init :70, feedInput* :164-205, PythonControl :240,
ExternSprintDatasetSource :325).
"""

from __future__ import annotations
import os
from typing import Any, Dict, List, Optional
import numpy

# names RASR looks up; kept in the spelling RASR uses
segmentOrderList: Optional[List[str]] = None
isInitialized = False
InputDim: Optional[int] = None
OutputDim: Optional[int] = None
sprintDataset: Optional["ExternSprintDatasetSource"] = None


class ExternSprintDatasetSource:
    """writes to the parent; the mirror image of the reader in ExternSprintDataset"""

    def __init__(self, c2p_fd: int, p2c_fd: int, input_dim: int, output_dim: int, num_segments: Optional[int]):
        self.pipe_c2p = os.fdopen(c2p_fd, "wb")
        self.pipe_p2c = os.fdopen(p2c_fd, "rb")
        self._send(("init", input_dim, output_dim, num_segments))

    def _send(self, msg):
        from returnn_b200.datasets.sprint import write_msg

        write_msg(self.pipe_c2p, msg)

    def add_new_data(self, segment_name: Optional[str], features: numpy.ndarray, targets: Dict[str, Any]):
        """one sequence; features [feature, time]"""
        self._send(("data", segment_name, features, targets))

    def close(self):
        """end of the epoch"""
        try:
            self._send(("exit",))
        finally:
            self.pipe_c2p.close()
            self.pipe_p2c.close()


def getSegmentList(corpusName, segmentList, **_kwargs):
    """PythonSegmentOrder hook: remembers the list (its length is announced to the parent), order unchanged"""
    global segmentOrderList
    segmentOrderList = list(segmentList)
    print("returnn_b200 extern_interface: corpus %r, %i segments" % (corpusName, len(segmentOrderList)))
    return segmentOrderList


def _parse_config(config: str) -> Dict[str, str]:
    """``key:value,key:value`` as given in ``--*.pymod-config``"""
    out = {}
    for item in config.split(","):
        if item:
            k, _, v = item.partition(":")
            out[k] = v
    return out


def _open_source(input_dim: int, output_dim: int, config: Dict[str, str]):
    global sprintDataset, isInitialized, InputDim, OutputDim
    assert config.get("action") == "ExternSprintDataset", "pymod-config must carry action:ExternSprintDataset, got %r" % (config,)
    InputDim, OutputDim = int(input_dim), int(output_dim)
    sprintDataset = ExternSprintDatasetSource(c2p_fd=int(config["c2p_fd"]), p2c_fd=int(config["p2c_fd"]), input_dim=InputDim,
                                              output_dim=OutputDim, num_segments=len(segmentOrderList) if segmentOrderList is not None else None)
    isInitialized = True


def init(name=None, sprint_unit=None, reference=None, config="", inputDim=None, outputDim=None, targetMode=None, **kwargs):
    """
    Called by RASR once. Two callers: the PythonTrainer (``inputDim`` / ``outputDim`` / ``targetMode`` given) and the generic
    PythonControl (``name`` / ``sprint_unit`` given, dimensions follow in ``init_processing``); the latter gets the class back.
    """
    cfg = _parse_config(config)
    if inputDim is not None:
        _open_source(inputDim, outputDim or 0, cfg)
        return None
    return PythonControl.create(config=cfg, name=name, sprint_unit=sprint_unit, **kwargs)


def exit():
    """called by RASR at its end"""
    global isInitialized
    if sprintDataset is not None and isInitialized:
        sprintDataset.close()
    isInitialized = False


def feedInput(features, weights=None, segmentName=None):
    """features only"""
    feedInputAndTarget(features=features, weights=weights, segmentName=segmentName)


def feedInputAndTargetAlignment(features, targetAlignment, weights=None, segmentName=None):
    """features and frame-wise alignment"""
    feedInputAndTarget(features=features, alignment=targetAlignment, weights=weights, segmentName=segmentName)


def feedInputAndTargetSegmentOrth(features, targetSegmentOrth, weights=None, segmentName=None):
    """features and orthography"""
    feedInputAndTarget(features=features, orthography=targetSegmentOrth, weights=weights, segmentName=segmentName)


def feedInputAndTarget(features, weights=None, segmentName=None, orthography=None, alignment=None, speaker_name=None, speaker_gender=None,
                       **kwargs):
    """the general form: whatever RASR knows about the segment"""
    assert isInitialized and sprintDataset is not None, "init() was not called"
    assert features.shape[0] == InputDim, "feature dim %i, expected %i" % (features.shape[0], InputDim)
    targets: Dict[str, Any] = {}
    if alignment is not None:
        targets["classes"] = numpy.asarray(alignment)
    if orthography is not None:
        targets["orth"] = orthography
    if speaker_name is not None:
        targets["speaker_name"] = speaker_name
    if speaker_gender is not None:
        targets["speaker_gender"] = speaker_gender
    sprintDataset.add_new_data(segment_name=segmentName, features=numpy.asarray(features), targets=targets)


class PythonControl:
    """the PythonControl flavour of the same thing: RASR calls ``init_processing`` / ``process_segment`` / ``exit``"""

    instance: Optional["PythonControl"] = None

    @classmethod
    def create(cls, **kwargs) -> "PythonControl":
        """one instance per process"""
        if cls.instance is None:
            cls.instance = cls(**kwargs)
        return cls.instance

    def __init__(self, config: Dict[str, str], **_kwargs):
        self.config = config

    def init_processing(self, input_dim, output_dim, **_kwargs):
        """dimensions are known now"""
        _open_source(input_dim, output_dim, self.config)

    def process_segment(self, name, orthography, features, alignment, soft_alignment, speaker_name=None, **_kwargs):
        """one segment"""
        assert soft_alignment is None, "soft alignments are not forwarded"
        feedInputAndTarget(features=features, segmentName=name, orthography=orthography, alignment=alignment, speaker_name=speaker_name)

    def exit(self, **_kwargs):
        """end"""
        exit()
