"""
Serving a model over HTTP (task ``search_server``) and dataset-wide output statistics (task ``analyze``).

Server: requests carry ONE sequence each (JSON arrays, or a WAV file body), the model's ``forward_step`` runs on batches that a
worker thread forms from whatever requests are waiting (up to ``web_server_max_batch``; a lone request is not held back), and
every request gets its own outputs back as JSON, sparse outputs also as text when a vocabulary is known. One thread owns the
model and the device; the HTTP threads only parse, enqueue and wait.

The reference offers both tasks for its graph-mode engine (returnn/__main__.py:695-711; returnn/tf/engine.py:2358 ``analyze``,
:2901 ``web_server``); here they run on the eager engine through the same ``forward_step`` that ``task = "forward"`` uses.

Request formats (POST to any path):

* ``Content-Type: application/json``: ``{"inputs": {"data": [[...], ...], ...}, "seq_tag": "optional"}``; a bare array is taken
  as the default input ``data``. Strings are encoded with the input's vocabulary.
* ``Content-Type: audio/wav`` (or ``audio/x-wav``): 16-bit PCM; fed as float samples in [-1, 1] of shape [T] or [T, 1] as the
  ``data`` template wants, or through ``ExtractAudioFeatures(**web_server_audio_opts)`` when that config key is set.

``GET /`` answers with the input / output templates. Config keys: ``web_server_port`` (12380), ``web_server_host`` (127.0.0.1),
``web_server_max_batch`` (16), ``web_server_batch_wait_ms`` (2: how long the worker waits for more requests once it has one).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Tuple
import io
import json
import queue
import threading
import time
import numpy
import torch

from ..log import log
from ..tensor import Tensor, TensorDict, batch_dim
from ..forward_iface import ForwardCallbackIface
from .. import frontend as rf

__all__ = ["ModelServer", "analyze", "FramewiseStatistics"]


# ---------------------------------------------------------------------------------------------------------------------
# serving


class _Collect(ForwardCallbackIface):
    def __init__(self):
        self.outputs: Dict[str, TensorDict] = {}

    def process_seq(self, *, seq_tag: str, outputs: TensorDict):
        self.outputs[seq_tag] = outputs


class _Request:
    __slots__ = ("inputs", "seq_tag", "done", "result", "error")

    def __init__(self, inputs: Dict[str, numpy.ndarray], seq_tag: str):
        self.inputs = inputs
        self.seq_tag = seq_tag
        self.done = threading.Event()
        self.result: Optional[Dict[str, Any]] = None
        self.error: Optional[str] = None


class ModelServer:
    """see the module docstring; ``serve_forever()`` blocks, ``start()`` / ``stop()`` run it in threads (used by the tests)"""

    def __init__(self, engine, *, port: int = 12380, host: str = "127.0.0.1", max_batch: int = 16, batch_wait_ms: float = 2.0):
        self.engine = engine
        self.config = engine.config
        self.max_batch = max(1, int(max_batch))
        self.batch_wait = max(0.0, float(batch_wait_ms)) / 1000.0
        self._queue: "queue.Queue[Optional[_Request]]" = queue.Queue()
        self._counter = 0
        self._counter_lock = threading.Lock()
        self._worker: Optional[threading.Thread] = None
        self._http_thread: Optional[threading.Thread] = None
        self.num_batches = 0
        self.num_requests = 0
        audio_opts = self.config.typed_value("web_server_audio_opts")
        self._audio_features = None
        if audio_opts:
            from ..datasets.util.feature_extraction import ExtractAudioFeatures

            self._audio_features = ExtractAudioFeatures(**audio_opts)
        self._httpd = self._make_httpd(host, port)
        self.port = self._httpd.server_address[1]

    # -- templates
    def _input_templates(self) -> Dict[str, Tensor]:
        return dict(self.engine.extern_data.data)

    def _vocab_of(self, t: Tensor):
        return getattr(t.sparse_dim, "vocab", None) if t.sparse_dim is not None else None

    def describe(self) -> Dict[str, Any]:
        """what ``GET /`` returns"""
        def one(t: Tensor):
            return {"dims": [d.dimension if not d.is_batch_dim() else "batch" for d in t.dims], "dtype": t.dtype,
                    "sparse_dim": t.sparse_dim.dimension if t.sparse_dim is not None else None, "has_vocab": self._vocab_of(t) is not None}

        out = {"inputs": {k: one(t) for k, t in self._input_templates().items() if k != "seq_tag"}, "epoch": self.engine.epoch,
               "max_batch": self.max_batch, "served_requests": self.num_requests, "served_batches": self.num_batches}
        model_outputs = self.config.typed_value("model_outputs")
        if isinstance(model_outputs, dict):
            out["outputs"] = sorted(model_outputs.keys())
        return out

    # -- request parsing
    def _next_tag(self) -> str:
        with self._counter_lock:
            self._counter += 1
            return "request-%i" % self._counter

    def parse_json(self, body: bytes) -> _Request:
        """JSON body -> request"""
        obj = json.loads(body.decode("utf8"))
        seq_tag = None
        if isinstance(obj, dict) and "inputs" in obj:
            seq_tag = obj.get("seq_tag")
            obj = obj["inputs"]
        if not isinstance(obj, dict):
            obj = {"data": obj}
        templates = self._input_templates()
        inputs = {}
        for key, value in obj.items():
            if key not in templates:
                raise ValueError("unknown input %r (the model takes %s)" % (key, sorted(k for k in templates if k != "seq_tag")))
            t = templates[key]
            if isinstance(value, str):
                vocab = self._vocab_of(t)
                if vocab is None:
                    raise ValueError("input %r was given as text, but it has no vocabulary" % key)
                value = vocab.get_seq(value)
            arr = numpy.asarray(value, dtype=t.dtype)
            if arr.ndim != len(t.dims) - 1:
                raise ValueError("input %r: expected %i axes (without batch), got shape %s" % (key, len(t.dims) - 1, arr.shape))
            inputs[key] = arr
        return _Request(inputs, seq_tag or self._next_tag())

    def parse_wav(self, body: bytes) -> _Request:
        """WAV body -> request for the default input"""
        import wave

        with wave.open(io.BytesIO(body), "rb") as w:
            if w.getsampwidth() != 2:
                raise ValueError("only 16-bit PCM WAV is handled, got sample width %i" % w.getsampwidth())
            rate, channels = w.getframerate(), w.getnchannels()
            pcm = numpy.frombuffer(w.readframes(w.getnframes()), dtype="<i2").astype("float32") / 32768.0
        if channels > 1:
            pcm = pcm.reshape(-1, channels).mean(axis=1)
        t = self._input_templates()["data"]
        if self._audio_features is not None:
            arr = self._audio_features.get_audio_features(pcm, rate).astype(t.dtype)
        elif len(t.dims) == 3:
            arr = pcm.astype(t.dtype)[:, None]
        else:
            arr = pcm.astype(t.dtype)
        return _Request({"data": arr}, self._next_tag())

    # -- the model side
    def _run_batch(self, requests: List[_Request]):
        from ..datasets.generating import StaticDataset

        try:
            tags = []
            for i, r in enumerate(requests):  # tags must be unique within the batch
                tags.append("%s#%i" % (r.seq_tag, i))
            dataset = StaticDataset(data=[dict(r.inputs, seq_tag=numpy.array(tag)) for r, tag in zip(requests, tags)])
            collect = _Collect()
            self.engine.forward_with_callback(dataset=dataset, callback=collect, allow_skipping_seqs=True)
            for r, tag in zip(requests, tags):
                outputs = collect.outputs.get(tag)
                if outputs is None:
                    r.error = "the model produced no output for this sequence"
                else:
                    r.result = self._encode_outputs(outputs)
        except Exception as exc:  # the server keeps running; every request of the batch learns why it failed
            import traceback

            print("search server: batch failed:\n%s" % traceback.format_exc(), file=log.v2)
            for r in requests:
                if r.result is None:
                    r.error = "%s: %s" % (type(exc).__name__, exc)
        finally:
            self.num_batches += 1
            self.num_requests += len(requests)
            for r in requests:
                r.done.set()

    def _encode_outputs(self, outputs: TensorDict) -> Dict[str, Any]:
        out = {}
        for key, t in outputs.data.items():
            arr = numpy.asarray(t.raw_tensor)
            out[key] = arr.tolist()
            vocab = self._vocab_of(t)
            if vocab is not None and arr.ndim == 1:
                out[key + ":text"] = vocab.get_seq_labels(arr)
        return out

    def _work(self):
        while True:
            first = self._queue.get()
            if first is None:
                return
            batch = [first]
            deadline = time.monotonic() + self.batch_wait
            stop = False
            while len(batch) < self.max_batch:
                timeout = deadline - time.monotonic()
                try:
                    nxt = self._queue.get(timeout=max(timeout, 0.0)) if timeout > 0 else self._queue.get_nowait()
                except queue.Empty:
                    break
                if nxt is None:
                    stop = True
                    break
                batch.append(nxt)
            self._run_batch(batch)
            if stop:
                return

    def submit(self, request: _Request, timeout: Optional[float] = None) -> Dict[str, Any]:
        """enqueue and wait (what the HTTP handler does)"""
        self._queue.put(request)
        if not request.done.wait(timeout):
            raise TimeoutError("no answer from the model within %r s" % timeout)
        if request.error is not None:
            raise RuntimeError(request.error)
        return request.result

    # -- HTTP
    def _make_httpd(self, host: str, port: int):
        from http.server import ThreadingHTTPServer, BaseHTTPRequestHandler

        server = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, fmt, *args):  # noqa
                print("search server: " + fmt % args, file=log.v4)

            def _send(self, code: int, obj):
                data = json.dumps(obj).encode("utf8")
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def do_GET(self):  # noqa
                self._send(200, server.describe())

            def do_POST(self):  # noqa
                try:
                    n = int(self.headers.get("Content-Length", "0"))
                    body = self.rfile.read(n)
                    ctype = (self.headers.get("Content-Type") or "application/json").split(";")[0].strip().lower()
                    if ctype in ("audio/wav", "audio/x-wav", "audio/wave"):
                        req = server.parse_wav(body)
                    else:
                        req = server.parse_json(body)
                except Exception as exc:
                    self._send(400, {"error": "%s: %s" % (type(exc).__name__, exc)})
                    return
                try:
                    result = server.submit(req, timeout=float(server.config.float("web_server_request_timeout", 600.0)))
                except Exception as exc:
                    self._send(500, {"error": str(exc), "seq_tag": req.seq_tag})
                    return
                self._send(200, {"seq_tag": req.seq_tag, "outputs": result})

        return ThreadingHTTPServer((host, port), Handler)

    def start(self):
        """worker and HTTP threads; returns at once"""
        self._worker = threading.Thread(target=self._work, name="search server model worker", daemon=True)
        self._worker.start()
        self._http_thread = threading.Thread(target=self._httpd.serve_forever, name="search server http", daemon=True)
        self._http_thread.start()

    def stop(self):
        """shut both threads down"""
        self._httpd.shutdown()
        self._httpd.server_close()
        self._queue.put(None)
        if self._worker is not None:
            self._worker.join(timeout=30)
        if self._http_thread is not None:
            self._http_thread.join(timeout=30)

    def serve_forever(self):
        """model worker in this thread's stead is not possible (the HTTP loop blocks), so: worker thread + HTTP loop here"""
        self._worker = threading.Thread(target=self._work, name="search server model worker", daemon=True)
        self._worker.start()
        print("search server: listening on %s:%i (max batch %i)" % (self._httpd.server_address[0], self.port, self.max_batch), file=log.v1)
        try:
            self._httpd.serve_forever()
        except KeyboardInterrupt:
            print("search server: interrupted", file=log.v1)
        finally:
            self._httpd.server_close()
            self._queue.put(None)
            self._worker.join(timeout=30)


# ---------------------------------------------------------------------------------------------------------------------
# analyze


class FramewiseStatistics(ForwardCallbackIface):
    """
    Accumulates over all sequences, from a per-frame class distribution (output ``analyze_output``, default ``"output"``: logits,
    log-probabilities or probabilities [T, V], told apart by their sums) and, when the dataset has it with one label per output
    frame, the target key (``analyze_target``, default ``"classes"``):

    ``frames``, ``seqs``, ``seq_len_{mean,min,max}``; ``entropy_mean`` (nats); ``max_prob_mean``; ``prior`` (average posterior per
    class) and ``argmax_histogram``; with targets: ``frame_error_rate``, ``ce_mean``, ``target_histogram``; with ``sil_label_idx``:
    the share of silence among targets and among decisions, and the frame error rate over non-silence frames.
    """

    def __init__(self, *, output_key: str = "output", target_key: Optional[str] = "classes", sil_label_idx: Optional[int] = None,
                 targets: Optional[Dict[str, numpy.ndarray]] = None, statistics: Optional[List[str]] = None):
        self.output_key = output_key
        self.target_key = target_key
        self.sil = sil_label_idx
        self.targets = targets or {}
        self.statistics = set(statistics) if statistics else None
        self.frames = 0
        self.seqs = 0
        self.lens: List[int] = []
        self.entropy_sum = 0.0
        self.max_prob_sum = 0.0
        self.prior_sum: Optional[numpy.ndarray] = None
        self.argmax_hist: Optional[numpy.ndarray] = None
        self.target_hist: Optional[numpy.ndarray] = None
        self.target_frames = 0
        self.errors = 0
        self.ce_sum = 0.0
        self.sil_target = 0
        self.sil_decision = 0
        self.non_sil_frames = 0
        self.non_sil_errors = 0

    @staticmethod
    def _log_probs(x: numpy.ndarray) -> numpy.ndarray:
        x = x.astype("float64")
        sums = x.sum(axis=-1)
        if (x >= 0).all() and numpy.allclose(sums, 1.0, atol=1e-3):
            return numpy.log(numpy.maximum(x, 1e-30))
        lse = numpy.log(numpy.exp(x - x.max(axis=-1, keepdims=True)).sum(axis=-1, keepdims=True)) + x.max(axis=-1, keepdims=True)
        return x - lse  # logits and log-probabilities alike (for the latter lse is 0)

    def process_seq(self, *, seq_tag: str, outputs: TensorDict):
        out = outputs.data[self.output_key]
        x = numpy.asarray(out.raw_tensor)
        assert x.ndim == 2, "analyze: output %r of a sequence must be [time, classes], got shape %s" % (self.output_key, x.shape)
        logp = self._log_probs(x)
        p = numpy.exp(logp)
        t, v = x.shape
        if self.prior_sum is None:
            self.prior_sum = numpy.zeros(v)
            self.argmax_hist = numpy.zeros(v, dtype="int64")
            self.target_hist = numpy.zeros(v, dtype="int64")
        self.frames += t
        self.seqs += 1
        self.lens.append(t)
        self.entropy_sum += float(-(p * logp).sum())
        self.max_prob_sum += float(p.max(axis=-1).sum())
        self.prior_sum += p.sum(axis=0)
        decision = p.argmax(axis=-1)
        self.argmax_hist += numpy.bincount(decision, minlength=v)
        if self.sil is not None:
            self.sil_decision += int((decision == self.sil).sum())
        target = None
        if self.target_key and self.target_key in outputs.data:
            target = numpy.asarray(outputs.data[self.target_key].raw_tensor)
        elif seq_tag in self.targets:
            target = self.targets[seq_tag]
        if target is not None and target.ndim == 1 and target.shape[0] == t:
            target = target.astype("int64")
            self.target_frames += t
            wrong = decision != target
            self.errors += int(wrong.sum())
            self.ce_sum += float(-logp[numpy.arange(t), target].sum())
            self.target_hist += numpy.bincount(target, minlength=v)
            if self.sil is not None:
                sil = target == self.sil
                self.sil_target += int(sil.sum())
                self.non_sil_frames += int((~sil).sum())
                self.non_sil_errors += int((wrong & ~sil).sum())

    def result(self) -> Dict[str, Any]:
        """the collected numbers"""
        n = max(self.frames, 1)
        res: Dict[str, Any] = {"frames": self.frames, "seqs": self.seqs}
        if self.lens:
            res.update(seq_len_mean=float(numpy.mean(self.lens)), seq_len_min=int(min(self.lens)), seq_len_max=int(max(self.lens)))
        if self.prior_sum is not None:
            res.update(entropy_mean=self.entropy_sum / n, max_prob_mean=self.max_prob_sum / n, prior=(self.prior_sum / n).tolist(),
                       argmax_histogram=self.argmax_hist.tolist())
        if self.target_frames:
            res.update(frame_error_rate=self.errors / self.target_frames, ce_mean=self.ce_sum / self.target_frames,
                       target_histogram=self.target_hist.tolist())
        if self.sil is not None:
            res["silence_share_decisions"] = self.sil_decision / n
            if self.target_frames:
                res["silence_share_targets"] = self.sil_target / self.target_frames
                res["frame_error_rate_non_silence"] = self.non_sil_errors / max(self.non_sil_frames, 1)
        if self.statistics is not None:
            res = {k: v for k, v in res.items() if k in self.statistics or k in ("frames", "seqs")}
        return res


def analyze(engine, data, statistics: Optional[List[str]] = None) -> Dict[str, Any]:
    """
    Run the model's ``forward_step`` over ``data`` and print / return :class:`FramewiseStatistics`.
    Targets come from the dataset (read once on the host, matched by sequence tag), so ``forward_step`` need not pass them on.
    """
    config = engine.config
    target_key = config.value("analyze_target", "classes")
    targets: Dict[str, numpy.ndarray] = {}
    if target_key and target_key in data.get_data_keys():
        data.init_seq_order(epoch=engine.epoch or 1)
        i = 0
        while data.is_less_than_num_seqs(i):
            data.load_seqs(i, i + 1)
            targets[data.get_tag(i)] = numpy.asarray(data.get_data(i, target_key))
            i += 1
    stats = FramewiseStatistics(output_key=config.value("analyze_output", "output"), target_key=target_key,
                                sil_label_idx=config.int("sil_label_idx", -1) if config.has("sil_label_idx") else None, targets=targets,
                                statistics=statistics)
    print("Analyze with the model on %r." % data, file=log.v1)
    start = time.monotonic()
    engine.forward_with_callback(dataset=data, callback=stats, allow_skipping_seqs=True)
    res = stats.result()
    print("Finished analyzing %r: %.1f s" % (data, time.monotonic() - start), file=log.v1)
    for k, v in sorted(res.items()):
        if isinstance(v, list) and len(v) > 20:
            v = "[%s, ... (%i values)]" % (", ".join("%.4g" % x for x in v[:10]), len(v))
        print("stats:%s: %s" % (k, v), file=log.v1)
    print("That are all collected stats.", file=log.v1)
    return res
