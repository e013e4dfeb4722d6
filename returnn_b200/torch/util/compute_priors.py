"""
``task = "compute_priors"``: average output distribution of the model over a dataset (the label prior that hybrid and
CTC decoders divide by).

``forward_step`` must mark an output (default name ``"output"``, config ``output_file_prior_key``) with a feature dim that holds
probabilities or log-probabilities (config ``priors_are_log``, default: values <= 0 everywhere are taken as logs). Padded
frames are excluded. The result is written as text: log priors to ``<output_file>`` (config ``output_file``, default
``priors.txt``), one number per class.

Parity: returnn/__main__.py:691-694 (task dispatch) and the prior computation of the engines (``compute_priors``).
"""

from __future__ import annotations
from typing import Optional
import numpy
import torch
from ...forward_iface import ForwardCallbackIface
from ...log import log


class _Accumulate(ForwardCallbackIface):
    def __init__(self, key: str, is_log: Optional[bool]):
        self.key = key
        self.is_log = is_log
        self.sum: Optional[numpy.ndarray] = None
        self.frames = 0

    def init(self, *, model):
        self.sum = None
        self.frames = 0

    def process_seq(self, *, seq_tag: str, outputs):
        out = outputs[self.key]
        raw = out.raw_tensor
        arr = raw.detach().float().cpu().numpy() if isinstance(raw, torch.Tensor) else numpy.asarray(raw, dtype="float32")
        feat_axis = out.feature_dim_axis if out.feature_dim_axis is not None else arr.ndim - 1
        arr = numpy.moveaxis(arr, feat_axis, -1).reshape(-1, arr.shape[feat_axis])
        is_log = self.is_log if self.is_log is not None else bool((arr <= 1e-6).all())
        probs = numpy.exp(arr.astype("float64")) if is_log else arr.astype("float64")
        self.sum = probs.sum(0) if self.sum is None else self.sum + probs.sum(0)
        self.frames += arr.shape[0]

    def finish(self):
        pass


def compute_priors(*, engine, dataset, config) -> numpy.ndarray:
    """
    :return: log priors [classes]; also written to the output file
    """
    key = config.value("output_file_prior_key", "output")
    is_log = config.typed_value("priors_are_log", None)
    cb = _Accumulate(key, is_log)
    engine.forward_with_callback(dataset=dataset, callback=cb, allow_skipping_seqs=True)
    assert cb.sum is not None and cb.frames > 0, "compute_priors: the dataset produced no frames"
    priors = cb.sum / cb.frames
    log_priors = numpy.log(numpy.maximum(priors, 1e-30))
    filename = config.value("output_file", "priors.txt")
    numpy.savetxt(filename, log_priors)
    print("compute_priors: %i frames, %i classes, sum of priors %.6f, written to %s" % (cb.frames, len(priors), float(priors.sum()), filename), file=log.v2)
    return log_priors
