"""
Tasks ``analyze`` and ``search_server`` (returnn_b200/torch/serving.py) on the CPU with the 12AX demo model:
statistics against a plain recomputation from the forward outputs, and HTTP requests (JSON and WAV bodies, concurrent clients
that the server batches) against direct forward results.
"""

import io
import json
import os
import threading
import urllib.request
import urllib.error
import numpy
import pytest
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(autouse=True)
def _masked_conv_behavior():
    """behaviour version 24: convolutions mask padded frames, so a sequence's result does not depend on what it is batched with"""
    from returnn_b200.utils.basic import BehaviorVersion

    BehaviorVersion._reset(24)
    yield
    BehaviorVersion._reset()


def _engine(tmp_path, **extra):
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.torch.engine import Engine
    from returnn_b200 import frontend as rf

    cfg = Config()
    cfg.load_file(os.path.join(_ROOT, "demos", "demo-rf.config"))
    cfg.update({"device": "cpu", "model": str(tmp_path / "model"), "learning_rate_file": str(tmp_path / "lr"), "log_verbosity": 3, "task": "forward"})
    cfg.update(extra)
    set_global_config(cfg)
    rf.select_backend_torch()
    torch.manual_seed(0)
    engine = Engine(cfg)
    engine.init_network_from_config(cfg)
    return engine, cfg


def test_analyze_statistics_match_a_recomputation(tmp_path):
    from returnn_b200.datasets.basic import init_dataset
    from returnn_b200.forward_iface import ForwardCallbackIface

    engine, cfg = _engine(tmp_path, sil_label_idx=0)
    data = init_dataset({"class": "Task12AXDataset", "num_seqs": 23, "fixed_random_seed": 3})
    res = engine.analyze(data=data, statistics=None)

    class Collect(ForwardCallbackIface):
        def __init__(self):
            self.out = {}

        def process_seq(self, *, seq_tag, outputs):
            self.out[seq_tag] = numpy.asarray(outputs["output"].raw_tensor)

    c = Collect()
    data2 = init_dataset({"class": "Task12AXDataset", "num_seqs": 23, "fixed_random_seed": 3})
    engine.forward_with_callback(dataset=data2, callback=c)
    data2.init_seq_order(epoch=1)
    frames = errors = sil_t = 0
    ce = 0.0
    prior = numpy.zeros(2)
    for i in range(23):
        data2.load_seqs(i, i + 1)
        logits = torch.from_numpy(c.out[data2.get_tag(i)]).double()
        target = torch.from_numpy(data2.get_data(i, "classes").astype("int64"))
        logp = torch.log_softmax(logits, dim=-1)
        frames += len(target)
        errors += int((logp.argmax(-1) != target).sum())
        ce += float(-logp[torch.arange(len(target)), target].sum())
        prior += logp.exp().sum(0).numpy()
        sil_t += int((target == 0).sum())
    assert res["frames"] == frames and res["seqs"] == 23
    assert abs(res["frame_error_rate"] - errors / frames) < 1e-9 and abs(res["ce_mean"] - ce / frames) < 1e-6
    assert numpy.allclose(res["prior"], prior / frames, atol=1e-6) and abs(sum(res["prior"]) - 1.0) < 1e-6
    assert abs(res["silence_share_targets"] - sil_t / frames) < 1e-9 and sum(res["target_histogram"]) == frames
    only = engine.analyze(data=init_dataset({"class": "Task12AXDataset", "num_seqs": 5}), statistics=["frame_error_rate"])
    assert set(only) == {"frames", "seqs", "frame_error_rate"}


def _post(port, body: bytes, ctype: str):
    req = urllib.request.Request("http://127.0.0.1:%i/" % port, data=body, headers={"Content-Type": ctype}, method="POST")
    with urllib.request.urlopen(req, timeout=120) as resp:
        return json.loads(resp.read().decode("utf8"))


def test_model_server_json_requests_are_batched_and_answered(tmp_path):
    from returnn_b200.torch.serving import ModelServer
    from returnn_b200.datasets.basic import init_dataset

    engine, cfg = _engine(tmp_path)
    server = ModelServer(engine, port=0, max_batch=8, batch_wait_ms=300)
    server.start()
    try:
        info = json.loads(urllib.request.urlopen("http://127.0.0.1:%i/" % server.port, timeout=30).read().decode("utf8"))
        assert info["inputs"]["data"]["dims"] == ["batch", None, 9] and info["outputs"] == ["output"]
        data = init_dataset({"class": "Task12AXDataset", "num_seqs": 6, "fixed_random_seed": 5})
        data.init_seq_order(epoch=1)
        seqs = []
        for i in range(6):
            data.load_seqs(i, i + 1)
            seqs.append(data.get_data(i, "data"))
        results = [None] * 6

        def client(i):
            results[i] = _post(server.port, json.dumps({"inputs": {"data": seqs[i].tolist()}, "seq_tag": "s%i" % i}).encode("utf8"), "application/json")

        threads = [threading.Thread(target=client, args=(i,)) for i in range(6)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
        assert server.num_requests == 6 and server.num_batches < 6  # concurrent requests shared batches
        model = engine._orig_model
        for i in range(6):
            assert results[i]["seq_tag"] == "s%i" % i
            got = numpy.array(results[i]["outputs"]["output"], dtype="float32")
            from returnn_b200.tensor import Tensor, Dim, batch_dim
            import returnn_b200.frontend as rf

            t = Dim(None, name="t")
            t.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([len(seqs[i])], dtype=torch.int32))
            x = Tensor("x", dims=[batch_dim, t, model.layers[0].in_dim], dtype="float32", raw_tensor=torch.from_numpy(seqs[i])[None])
            rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)
            with torch.no_grad():
                ref = model(x, spatial_dim=t).copy_transpose([batch_dim, t, model.layers[-1].out_dim]).raw_tensor[0].numpy()
            assert got.shape == ref.shape and numpy.allclose(got, ref, atol=1e-5)
        # a bare array is the default input; malformed requests get a 400 with the reason, the server keeps serving
        bare = _post(server.port, json.dumps(seqs[0].tolist()).encode("utf8"), "application/json")
        assert numpy.allclose(numpy.array(bare["outputs"]["output"]), numpy.array(results[0]["outputs"]["output"]), atol=1e-6)
        for bad in (b"{not json", json.dumps({"inputs": {"nope": [1]}}).encode(), json.dumps({"inputs": {"data": [1.0, 2.0]}}).encode()):
            with pytest.raises(urllib.error.HTTPError) as exc_info:
                _post(server.port, bad, "application/json")
            assert exc_info.value.code == 400 and "error" in json.loads(exc_info.value.read().decode("utf8"))
        again = _post(server.port, json.dumps(seqs[1].tolist()).encode("utf8"), "application/json")
        assert len(again["outputs"]["output"]) == len(seqs[1])
    finally:
        server.stop()


def test_model_server_wav_body(tmp_path):
    import wave
    from returnn_b200.torch.serving import ModelServer

    engine, cfg = _engine(tmp_path, web_server_audio_opts={"features": "mfcc", "num_feature_filters": 9, "window_len": 0.025, "step_len": 0.01})
    server = ModelServer(engine, port=0)
    server.start()
    try:
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(1)
            w.setsampwidth(2)
            w.setframerate(16000)
            w.writeframes((numpy.sin(numpy.arange(8000) * 0.03) * 12000).astype("<i2").tobytes())
        res = _post(server.port, buf.getvalue(), "audio/wav")
        out = numpy.array(res["outputs"]["output"])
        assert out.ndim == 2 and out.shape[1] == 2 and 40 <= out.shape[0] <= 52 and numpy.isfinite(out).all()
    finally:
        server.stop()
