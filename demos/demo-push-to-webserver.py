#!/usr/bin/env python3
"""
Client of ``task = "search_server"``: sends feature arrays (or a WAV file) to a running server and prints the answer.

    python rnn.py my.config ++task search_server ++web_server_port 12380 &
    python demos/demo-push-to-webserver.py --port 12380                      # random features of the right shape
    python demos/demo-push-to-webserver.py --port 12380 --wav utterance.wav  # needs web_server_audio_opts in the config

Without ``--port`` the script starts a server around a tiny model in this process first (nothing else needed) and talks to that.
"""

import argparse
import json
import urllib.request
import _setup_env  # noqa: F401
import numpy


def _tiny_server():
    import torch
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Dim, batch_dim
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.torch.engine import Engine

    time_dim, feat, out = Dim(None, name="time"), Dim(9, name="feat"), Dim(2, name="out")

    class Model(rf.Module):
        def __init__(self):
            super().__init__()
            self.lin = rf.Linear(feat, out)

        def __call__(self, x):
            return rf.softmax(self.lin(x), axis=out)

    def forward_step(*, model, extern_data, **_kw):
        y = model(extern_data["data"])
        y.mark_as_default_output(shape=[batch_dim, time_dim, out])

    cfg = Config({"task": "search_server", "backend": "torch", "device": "cpu", "behavior_version": 24,
                  "extern_data": {"data": {"dims": [batch_dim, time_dim, feat], "dtype": "float32"}}, "get_model": lambda **_kw: Model(),
                  "forward_step": forward_step, "web_server_port": 0, "log_verbosity": 3, "batch_size": 10000, "max_seqs": 16})
    set_global_config(cfg)
    torch.manual_seed(0)
    from returnn_b200.torch.serving import ModelServer

    engine = Engine(cfg)
    engine.init_network_from_config(cfg)
    server = ModelServer(engine, port=0)
    server.start()
    return server


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int)
    ap.add_argument("--wav")
    ap.add_argument("--frames", type=int, default=7)
    ap.add_argument("--dim", type=int, default=9)
    args = ap.parse_args()
    server = None
    if args.port is None:
        server = _tiny_server()
        args.port = server.port
        print("started a server around a tiny model on port", args.port)
    url = "http://%s:%i/" % (args.host, args.port)
    if args.wav:
        req = urllib.request.Request(url, data=open(args.wav, "rb").read(), headers={"Content-Type": "audio/wav"})
    else:
        feats = numpy.random.RandomState(1).randn(args.frames, args.dim).astype("float32")
        req = urllib.request.Request(url, data=json.dumps({"data": feats.tolist()}).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=60) as resp:
        answer = json.loads(resp.read())
    print("seq_tag:", answer.get("seq_tag"))
    for k, v in (answer.get("outputs") or {}).items():
        arr = numpy.asarray(v) if isinstance(v, list) else v
        print("output %r:" % k, getattr(arr, "shape", ""), arr if not hasattr(arr, "shape") or arr.size <= 20 else "...")
    if "error" in answer:
        print("error:", answer["error"])
    if server is not None:
        server.stop()


if __name__ == "__main__":
    main()
