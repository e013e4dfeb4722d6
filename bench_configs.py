#!/usr/bin/env python3
"""
Training throughput of the other baseline configurations (the flagship Conformer-CTC has its own ``bench.py``), through the
public engine API on synthetic data of the named shapes with random-init weights:

    python bench_configs.py --config blstm_ctc       # 6 x BLSTM(1024) + CTC, 20k frames per batch, AdamW
    python bench_configs.py --config conformer_aed   # 12-layer Conformer + 6-layer Transformer decoder, CE + aux CTC
    python bench_configs.py --config transformer_mt  # Transformer base, shared 32k vocabulary, 25k tokens per batch
    python bench_configs.py --config 12ax            # 2 x BLSTM(100) on the 12AX task, CPU fp32, 2 epochs x 1000 seqs (wall time)

One JSON line per run: device-timed (CUDA events around K steps after W warm-up steps), a distinct batch every step, inputs
staged on the device for ``value`` and copied from pinned host memory inside the timed region for ``e2e``. Multi-GPU:
launch with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench_configs.py --config ... --gpus N``.
"""

from __future__ import annotations
import argparse
import json
import os
import sys
import time

_ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, _ROOT)
import bench as _bench  # noqa: E402  (batch synthesis, collate, clock sampler)

FRAME_SEC = 0.01


def _asr_batches(seed, n_steps, frames_budget, min_len, max_len, label_ratio):
    """80-dim features ~N(0,1), labels uniform over 1..9999 with length ratio * frames (a pair: uniform in the range)"""
    import numpy

    rng = numpy.random.RandomState(seed)
    batches, cur, cur_max = [], [], 0
    while len(batches) < n_steps:
        t = int(rng.randint(min_len, max_len + 1))
        r = rng.uniform(*label_ratio) if isinstance(label_ratio, tuple) else label_ratio
        s = max(1, int(round(t * r)))
        seq = {"data": rng.standard_normal((t, 80)).astype("float32"), "classes": rng.randint(1, 10000, size=(s,)).astype("int32")}
        new_max = max(cur_max, t)
        if cur and new_max * (len(cur) + 1) > frames_budget:
            batches.append(cur)
            cur, cur_max = [seq], t
        else:
            cur.append(seq)
            cur_max = new_max
    return batches


def _mt_batches(seed, n_steps, tokens_budget, vocab=32000):
    """token ids Zipf(1.1) over the vocabulary, source length 10..100, target length = source * U(0.8, 1.2)"""
    import numpy

    rng = numpy.random.RandomState(seed)
    ranks = numpy.arange(1, vocab, dtype="float64")
    probs = ranks ** -1.1
    probs /= probs.sum()
    cdf = numpy.cumsum(probs)

    def draw(n):
        return (numpy.searchsorted(cdf, rng.random_sample(n)) + 1).clip(1, vocab - 1).astype("int32")

    batches, cur, cur_max = [], [], 0
    while len(batches) < n_steps:
        s = int(rng.randint(10, 101))
        t = max(1, int(round(s * rng.uniform(0.8, 1.2))))
        seq = {"data": draw(s), "classes": draw(t)}
        new_max = max(cur_max, s, t)
        if cur and new_max * (len(cur) + 1) > tokens_budget:
            batches.append(cur)
            cur, cur_max = [seq], max(s, t)
        else:
            cur.append(seq)
            cur_max = new_max
    return batches


def _ref_hook(state, W, K, counts, meta):
    """
    Timing hook of the reference-arm configs, called at the start of their ``train_step``: at steps W and W+K the device is
    synchronised, the ranks are aligned and a CUDA event is recorded; after the second one rank 0 prints the JSON line (time =
    max over ranks, counts summed over ranks).
    """
    import torch

    n = state["n"]
    state["n"] = n + 1
    if n != W and n != W + K:
        return
    torch.cuda.synchronize()
    dist_on = torch.distributed.is_available() and torch.distributed.is_initialized()
    if dist_on:
        torch.distributed.barrier()
        torch.cuda.synchronize()
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    if n == W:
        state["ev0"] = ev
        return
    torch.cuda.synchronize()
    ms = state["ev0"].elapsed_time(ev)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    f = torch.tensor([float(sum(counts[W:W + K]))], device="cuda", dtype=torch.float64)
    world = 1
    if dist_on:
        world = torch.distributed.get_world_size()
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(f, op=torch.distributed.ReduceOp.SUM)
    if int(os.environ.get("RANK", "0")) == 0:
        out = {"impl": "reference", "metric": meta["metric"], "value": f.item() * meta.get("count_scale", 1.0) / (t.item() / 1e3), "unit": meta["unit"],
               "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": t.item() / K, "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
               "data": "synthetic", "config": {"model": meta["model"], "parallelism": meta.get("parallelism", "dp%i" % world)}}
        sys.__stdout__.write(json.dumps(out) + "\n")
        sys.__stdout__.flush()



def _configs():
    from returnn_b200.models import blstm_ctc, conformer_aed, transformer_mt

    return {
        "blstm_ctc": dict(
            mod=blstm_ctc, model_opts={}, name="blstm-ctc 6x1024 (2x time reduction after layers 1 and 2) vocab10k",
            batches=lambda seed, n: _asr_batches(seed, n, 20000, 500, 1600, (0.1, 0.25)), budget=20000, unit="audio-s/s",
            metric="train seconds-of-audio per second", output_dim={"data": (80, 2), "classes": (10000, 1)}, count=lambda b: sum(s["data"].shape[0] for s in b) * FRAME_SEC,
            extra={"optimizer": {"class": "adamw", "weight_decay": 0.01}}),
        "conformer_aed": dict(
            mod=conformer_aed, model_opts={}, name="conformer-aed 12x512 + 6-layer decoder, CE(ls 0.1) + 0.3 CTC, vocab10k",
            batches=lambda seed, n: _asr_batches(seed, n, 40000, 300, 2000, 1.0 / 30.0), budget=40000, unit="audio-s/s",
            metric="train seconds-of-audio per second", output_dim={"data": (80, 2), "classes": (10000, 1)}, count=lambda b: sum(s["data"].shape[0] for s in b) * FRAME_SEC,
            extra={"optimizer": {"class": "adamw", "weight_decay": 0.01}, "gradient_clip_global_norm": 5.0}),
        "transformer_mt": dict(
            mod=transformer_mt, model_opts={}, name="transformer-base 6+6x512 h8 ff2048 shared vocab 32k",
            batches=lambda seed, n: _mt_batches(seed, n, 25000), budget=25000, unit="tokens/s", metric="train tokens per second (source + target)",
            output_dim={"data": (32000, 1), "classes": (32000, 1)}, count=lambda b: sum(s["data"].shape[0] + s["classes"].shape[0] for s in b),
            extra={"optimizer": {"class": "adamw", "betas": (0.9, 0.98), "eps": 1e-9, "weight_decay": 0.0}}),
    }


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.log import log
    from returnn_b200.utils.basic import BehaviorVersion
    from returnn_b200.torch.engine import Engine
    from returnn_b200.datasets.generating import StaticDataset
    from returnn_b200.ops import _lib

    spec = _configs()[args.config]
    rank, world, local_rank = _bench._dist_env()
    assert world == args.gpus
    torch.cuda.set_device(local_rank)
    W, K = args.warmup, args.steps
    # a pool of distinct batches that is walked round and round: consecutive steps never see the same batch and the pool (> 200 MB
    # of inputs) exceeds the L2, while a 100-step run does not pin gigabytes of host memory
    n_pool = 2 * (W + K) + 3 if args.task == "search" else min(2 * (W + K) + 3, 24)
    batches = spec["batches"](4321 + rank, n_pool)
    mod = spec["mod"]
    cfg = Config(dict({
        "task": "train", "backend": "torch", "behavior_version": 24, "extern_data": mod.make_extern_data(spec["model_opts"]),
        "model_opts": dict(spec["model_opts"]), "get_model": mod.get_model, "train_step": mod.train_step, "batch_size": spec["budget"],
        "max_seqs": 2000, "learning_rate": 1e-4, "torch_amp": "bfloat16", "num_epochs": 1, "log_verbosity": 2 if rank == 0 else 1,
        "device": "cuda", "forward_step": getattr(mod, "forward_step", None)}, **spec["extra"]))
    if world > 1:
        cfg.set("torch_distributed", {"reduce_type": "param", "param_sync_step": 100} if args.config == "conformer_aed" else
                {"reduce_type": "grad_explicit" if args.cuda_graph else "grad"})
    if args.graph_decoder:
        # decoder + loss of the encoder-decoder model as a captured forward / backward graph pair, bounded by the largest batch of the pool
        assert args.config == "conformer_aed"
        enc_len = lambda t: -(-(-(-t // 3)) // 2)
        cfg.set("model_opts", dict(spec["model_opts"], graphed_decoder={
            "batch_size_bound": max(len(b) for b in batches), "enc_capacity": -(-enc_len(max(s["data"].shape[0] for b in batches for s in b)) // 8) * 8,
            "tgt_capacity": -(-max(s["classes"].shape[0] for b in batches for s in b) // 8) * 8}))
    if args.cuda_graph:
        # whole-step graph replay over buffers bounded by the largest batch of the pool (sequences, and frames per key rounded up to 8)
        cap = {k: -(-max(s[k].shape[0] for b in batches for s in b) // 8) * 8 for k in ("data", "classes")}
        cfg.set("torch_cuda_graph", {"batch_size_bound": max(len(b) for b in batches), "dim_capacity": cap, "warmup_steps": 2})
    set_global_config(cfg)
    BehaviorVersion._reset(24)
    log.init_by_config(cfg)
    train_data = StaticDataset(data=[s for b in batches[:2] for s in b], output_dim=spec["output_dim"])
    train_data.initialize()
    engine = Engine(cfg)
    engine.init_train_from_config(cfg, train_data, None, None)
    engine.epoch = 1
    engine._pt_model.train()
    dev = torch.device("cuda", local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    raws = [_bench._collate(b, pin=True) for b in batches]
    counts = [spec["count"](b) for b in batches]

    def to_dev(raw):
        out = dict(raw)
        for k in ("data", "classes"):
            out[k] = raw[k].to(dev, non_blocking=True)
        return out

    if args.task == "search":
        # beam search through forward_step (beam size and length limit from the model options), end to end per batch: pinned host
        # batch -> device, decode, best hypotheses and their lengths back on the host
        from returnn_b200.torch.data import extern_data as extern_data_util
        import returnn_b200.frontend as rf

        engine._pt_model.eval()
        n_hyp_tokens = 0

        def decode(raw):
            extern = extern_data_util.raw_dict_to_extern_data(raw, extern_data_template=engine.extern_data, device=engine._device,
                                                              float_dtype=engine._default_float_dtype, with_eval_targets=False)
            engine._run_step(extern, train_func=False)
            out = rf.get_run_ctx().outputs["output"]
            hyp = out.raw_tensor.cpu()
            lens = out.dims[1].dyn_size_ext.raw_tensor.cpu()
            return hyp, lens

        with torch.no_grad():
            for i in range(W):
                decode(raws[i])
            barrier()
            sampler = _bench.ClockSampler(local_rank)
            if rank == 0:
                sampler.start()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(K):
                hyp, lens = decode(raws[W + i])
                n_hyp_tokens += int(lens.sum())
            ev1.record()
            barrier()
        ms = ev0.elapsed_time(ev1)
        clocks = sampler.stop() if rank == 0 else None
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        f = torch.tensor([sum(counts[W: W + K])], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(f, op=dist.ReduceOp.SUM)
        if rank == 0:
            print(json.dumps({"metric": "beam search " + spec["metric"].replace("train ", ""), "value": f.item() / (t.item() / 1e3), "unit": spec["unit"],
                              "n_gpus": world, "steps": K, "warmup": W, "ms_per_batch": t.item() / K, "higher_is_better": True, "dtype": "bf16",
                              "data": "synthetic", "impl": "returnn_b200", "config": {"model": spec["name"], "batch": "%i per GPU" % spec["budget"],
                                                                                          "beam_size": getattr(engine._orig_model, "beam_size", None),
                                                                                          "hyp_tokens_per_batch": n_hyp_tokens / K},
                              "clocks": clocks}))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    for i in range(W):
        engine.run_train_step(to_dev(raws[i % n_pool]), read_losses=False)
    staged = [to_dev(raws[(W + i) % n_pool]) for i in range(min(K, n_pool))]
    barrier()
    sampler = _bench.ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(K):
        engine.run_train_step(staged[i % len(staged)], read_losses=False)
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = _lib.launch_count() - launches0
    del staged
    base = W + K
    for i in range(3):
        engine.run_train_step(raws[(base + i) % n_pool], read_losses=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h2d = 0
    last = None
    for i in range(K):
        raw = raws[(base + 3 + i) % n_pool]
        h2d += raw["data"].numel() * raw["data"].element_size() + raw["classes"].numel() * raw["classes"].element_size()
        last = engine.run_train_step(raw, read_losses=True)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
    f = torch.tensor([sum(counts[(W + i) % n_pool] for i in range(K)), sum(counts[(base + 3 + i) % n_pool] for i in range(K))], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
    dev_ms, e2e_ms = t.tolist()
    n_dev, n_e2e = f.tolist()
    if rank == 0:
        print(json.dumps({
            "metric": spec["metric"], "value": n_dev / (dev_ms / 1e3), "unit": spec["unit"], "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "returnn_b200", "config": {"model": spec["name"], "global_batch": "%i per GPU x %i" % (spec["budget"], world),
                                                "parallelism": ("dp%i param averaging every 100 steps" % world) if args.config == "conformer_aed" else "dp%i" % world},
            "grad_reduce": engine._torch_distributed_ctx.grad_reduce_mode if engine._torch_distributed_ctx else "none",
            "cuda_graph": bool(args.cuda_graph), "graph_decoder": bool(args.graph_decoder), "clocks": clocks, "e2e": {"value": n_e2e / (e2e_ms / 1e3), "unit": spec["unit"], "ms_per_step": e2e_ms / K, "h2d_bytes_per_step": h2d // K,
                                      "d2h_bytes_per_step": 4 * max(len(last or {}), 1), "last_loss": last},
            "gpu_launches": launches}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_12ax(args):
    """config 1: CPU, fp32, 2 epochs x 1000 sequences, wall time and final dev frame error"""
    import torch
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.log import log
    from returnn_b200.datasets.basic import init_dataset
    from returnn_b200.torch.engine import Engine
    from returnn_b200.tensor import Dim, batch_dim
    import returnn_b200.frontend as rf

    torch.set_num_threads(int(os.environ.get("OMP_NUM_THREADS", "8")))
    time_dim, in_dim, out_dim = Dim(None, name="time"), Dim(9, name="in"), Dim(2, name="out")

    class Model(rf.Module):
        def __init__(self):
            super().__init__()
            h = Dim(100, name="lstm")
            h2 = 2 * h
            self.fw1, self.bw1 = rf.LSTM(in_dim, h), rf.LSTM(in_dim, h)
            self.fw2, self.bw2 = rf.LSTM(h2, h), rf.LSTM(h2, h)
            self.out = rf.Linear(h2, out_dim)
            self.h2 = h2

        def _bi(self, fw, bw, x, out_feat):
            y1, _ = fw(x, state=fw.default_initial_state(batch_dims=[batch_dim]), spatial_dim=time_dim)
            xr = rf.reverse_sequence(x, axis=time_dim)
            y2, _ = bw(xr, state=bw.default_initial_state(batch_dims=[batch_dim]), spatial_dim=time_dim)
            y2 = rf.reverse_sequence(y2, axis=time_dim)
            y, _ = rf.concat((y1, y1.feature_dim), (y2, y2.feature_dim), out_dim=out_feat)
            return y

        def __call__(self, x):
            y = self._bi(self.fw1, self.bw1, x, self.h2)
            y = self._bi(self.fw2, self.bw2, y, self.h2)
            return self.out(y)

    def train_step(*, model, extern_data, **_):
        logits = model(extern_data["data"])
        targets = extern_data["classes"]
        rf.cross_entropy(estimated=logits, estimated_type="logits", target=targets, axis=out_dim).mark_as_loss("ce")
        rf.cast(rf.reduce_argmax(logits, axis=out_dim) != targets, "float32").mark_as_loss("fer", as_error=True)

    config = Config({
        "backend": "torch", "task": "train", "num_epochs": 2, "batch_size": 5000, "max_seqs": 1000, "optimizer": {"class": "adam"},
        "learning_rate": 1e-3, "device": "cpu", "log_verbosity": 2,
        "extern_data": {"data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"},
                        "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32"}},
        "get_model": lambda **_: Model(), "train_step": train_step})
    set_global_config(config)
    log.init_by_config(config)
    train = init_dataset({"class": "Task12AXDataset", "num_seqs": 1000})
    dev = init_dataset({"class": "Task12AXDataset", "num_seqs": 100, "fixed_random_seed": 1})
    engine = Engine(config)
    engine.init_train_from_config(config, train, dev, None)
    t0 = time.perf_counter()
    engine.train()
    wall = time.perf_counter() - t0
    scores = engine.learning_rate_control.epoch_data[engine.epoch].error
    print(json.dumps({"metric": "12AX 2xBLSTM(100) CPU fp32: wall seconds for 2 epochs x 1000 seqs", "value": wall, "unit": "s", "higher_is_better": False,
                      "impl": "returnn_b200", "dtype": "fp32", "data": "synthetic (Task12AXDataset)", "final_scores": scores,
                      "threads": torch.get_num_threads()}))


_REF_12AX_CONFIG = r'''#!rnn.py
import time
from returnn.tensor import Tensor, Dim, batch_dim, TensorDict
import returnn.frontend as rf

backend = "torch"
task = "train"
device = "cpu"
train = {"class": "Task12AXDataset", "num_seqs": 1000}
dev = {"class": "Task12AXDataset", "num_seqs": 100, "fixed_random_seed": 1}
time_dim = Dim(None, name="time")
in_dim = Dim(9, name="in")
out_dim = Dim(2, name="out")
extern_data = {
    "data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"},
    "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32", "available_for_inference": False},
}
batch_size = 5000
max_seqs = 1000
optimizer = {"class": "adam"}
learning_rate = 1e-3
num_epochs = 2
log_verbosity = 3
torch_dataloader_opts = {"num_workers": 0}


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        h = Dim(100, name="lstm")
        self.h2 = 2 * h
        self.fw1, self.bw1 = rf.LSTM(in_dim, h), rf.LSTM(in_dim, h)
        self.fw2, self.bw2 = rf.LSTM(self.h2, h), rf.LSTM(self.h2, h)
        self.out = rf.Linear(self.h2, out_dim)

    def _bi(self, fw, bw, x):
        y1, _ = fw(x, state=fw.default_initial_state(batch_dims=[batch_dim]), spatial_dim=time_dim)
        xr = rf.reverse_sequence(x, axis=time_dim)
        y2, _ = bw(xr, state=bw.default_initial_state(batch_dims=[batch_dim]), spatial_dim=time_dim)
        y2 = rf.reverse_sequence(y2, axis=time_dim)
        y, _ = rf.concat((y1, y1.feature_dim), (y2, y2.feature_dim), out_dim=self.h2)
        return y

    def __call__(self, x):
        return self.out(self._bi(self.fw2, self.bw2, self._bi(self.fw1, self.bw1, x)))


def get_model(**_kwargs):
    return Model()


def train_step(*, model, extern_data, **_kwargs):
    logits = model(extern_data["data"]).copy_transpose((batch_dim, time_dim, out_dim))
    targets = extern_data["classes"]
    rf.cross_entropy(estimated=logits, estimated_type="logits", target=targets, axis=out_dim).mark_as_loss("ce")
    rf.cast(rf.reduce_argmax(logits, axis=out_dim) != targets, "float32").mark_as_loss("fer", as_error=True)
'''


_REF_MT_CONFIG = r'''#!rnn.py
import os, sys, time, json
import numpy, torch
from returnn.tensor import Tensor, Dim, batch_dim, TensorDict
import returnn.frontend as rf
from returnn.frontend.encoder.transformer import TransformerEncoder
from returnn.frontend.decoder.transformer import TransformerDecoder

_opts = __OPTS__
sys.path.insert(0, _opts["root"])
import bench_configs as _bc

backend = "torch"
task = "train"
behavior_version = 24
_W, _K = _opts["warmup"], _opts["steps"]
_rank, _world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
_batches = _bc._mt_batches(4321 + _rank, _W + _K + 1, 25000)
_parallelism = "dp%i" % _world
if _world > 1:
    torch_distributed = {"reduce_type": "grad"}
_tokens = [sum(s["data"].shape[0] + s["classes"].shape[0] for s in b) for b in _batches]
train = {"class": "StaticDataset", "data": [s for b in _batches for s in b], "output_dim": {"data": (32000, 1), "classes": (32000, 1)}}
src_time = Dim(None, name="src-time", kind=Dim.Types.Spatial)
tgt_time = Dim(None, name="tgt-time", kind=Dim.Types.Spatial)
vocab_dim = Dim(32000, name="vocab", kind=Dim.Types.Feature)
extern_data = {
    "data": {"dims": (batch_dim, src_time), "sparse_dim": vocab_dim, "dtype": "int32"},
    "classes": {"dims": (batch_dim, tgt_time), "sparse_dim": vocab_dim, "dtype": "int32", "available_for_inference": False},
}
batch_size = 25000
max_seqs = 2000
batching = "default"
optimizer = {"class": "adamw", "betas": (0.9, 0.98), "epsilon": 1e-9, "weight_decay": 0.0}
learning_rate = 1e-4
torch_amp = "bfloat16"
num_epochs = 1
log_verbosity = 3
torch_dataloader_opts = {"num_workers": 0}


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        md = Dim(512, name="model")
        self.encoder = TransformerEncoder(vocab_dim, md, num_layers=6, num_heads=8, dropout=0.1, att_dropout=0.1)
        self.decoder = TransformerDecoder(md, vocab_dim, Dim(512, name="dec-model"), num_layers=6, num_heads=8, ff_dim=Dim(2048, name="dec-ff"),
                                          dropout=0.1, att_dropout=0.1, share_embedding=True)


def get_model(**_kwargs):
    return Model()


_state = {"n": 0, "ev0": None}


def train_step(*, model, extern_data, **_kwargs):
    _bc._ref_hook(_state, _W, _K, _tokens, {"metric": "train tokens per second (source + target)", "unit": "tokens/s", "model": "transformer-base 6+6x512 h8 ff2048 shared vocab 32k (reference rf modules)", "count_scale": 1.0, "parallelism": _parallelism})
    src, tgt = extern_data["data"], extern_data["classes"]
    enc = model.encoder(src, spatial_dim=src_time)
    inp, (tgt_ext,) = rf.pad(tgt, axes=[tgt_time], padding=[(1, 0)], value=0)
    out_t, _ = rf.pad(tgt, axes=[tgt_time], padding=[(0, 1)], value=0, out_dims=[tgt_ext], handle_dynamic_dims=True)
    enc_state = model.decoder.transform_encoder(enc, axis=src_time)
    logits, _ = model.decoder(inp, spatial_dim=tgt_ext, encoder=enc_state, state=model.decoder.default_initial_state(batch_dims=[batch_dim]))
    log_prob = rf.log_softmax(logits, axis=vocab_dim)
    log_prob = rf.label_smoothed_log_prob_gradient(log_prob, 0.1, axis=vocab_dim)
    ce = rf.cross_entropy(target=out_t, estimated=log_prob, estimated_type="log-probs", axis=vocab_dim)
    ce.mark_as_loss("ce", use_normalized_loss=True)
    err = rf.reduce_argmax(logits, axis=vocab_dim) != out_t
    err.mark_as_loss("fer", as_error=True)
'''


_REF_AED_CONFIG = r'''#!rnn.py
import os, sys, time, json
import numpy, torch
from returnn.tensor import Tensor, Dim, batch_dim, TensorDict
import returnn.frontend as rf
from returnn.frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample
from returnn.frontend.decoder.transformer import TransformerDecoder

_opts = __OPTS__
sys.path.insert(0, _opts["root"])
import bench_configs as _bc

backend = "torch"
task = "train"
behavior_version = 24
_W, _K = _opts["warmup"], _opts["steps"]
_rank, _world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
_batches = _bc._asr_batches(4321 + _rank, _W + _K + 1, 40000, 300, 2000, 1.0 / 30.0)
_parallelism = "dp%i param averaging every 100 steps" % _world
if _world > 1:
    torch_distributed = {"reduce_type": "param", "param_sync_step": 100}
_frames = [sum(s["data"].shape[0] for s in b) for b in _batches]
train = {"class": "StaticDataset", "data": [s for b in _batches for s in b], "output_dim": {"data": (80, 2), "classes": (10000, 1)}}
time_dim = Dim(None, name="time", kind=Dim.Types.Spatial)
feat_dim = Dim(80, name="feature", kind=Dim.Types.Feature)
targets_time = Dim(None, name="targets-time", kind=Dim.Types.Spatial)
vocab_dim = Dim(10000, name="vocab", kind=Dim.Types.Feature)
extern_data = {
    "data": {"dims": (batch_dim, time_dim, feat_dim), "dtype": "float32"},
    "classes": {"dims": (batch_dim, targets_time), "sparse_dim": vocab_dim, "dtype": "int32", "available_for_inference": False},
}
batch_size = 40000
max_seqs = 2000
batching = "default"
optimizer = {"class": "adamw", "weight_decay": 0.01}
learning_rate = 1e-4
gradient_clip_global_norm = 5.0
torch_amp = "bfloat16"
num_epochs = 1
log_verbosity = 3
torch_dataloader_opts = {"num_workers": 0}


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        self.model_dim = Dim(512, name="enc-model")
        self.encoder = ConformerEncoder(
            feat_dim, self.model_dim, num_layers=12, num_heads=8, ff_dim=Dim(2048, name="enc-ff"), conv_kernel_size=32, dropout=0.1, att_dropout=0.1,
            conv_norm=rf.build_dict(rf.BatchNorm, use_mask=True),
            input_layer=ConformerConvSubsample(feat_dim, out_dims=[Dim(32, name="conv1"), Dim(64, name="conv2"), Dim(64, name="conv3")],
                                               filter_sizes=[(3, 3), (3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)]))
        self.decoder = TransformerDecoder(encoder_dim=self.model_dim, vocab_dim=vocab_dim, model_dim=Dim(512, name="dec-model"), num_layers=6,
                                          num_heads=8, ff_dim=Dim(2048, name="dec-ff"), dropout=0.1, att_dropout=0.1)
        self.wb_vocab_dim = vocab_dim + 1
        self.aux_ctc = rf.Linear(self.model_dim, self.wb_vocab_dim)


def get_model(**_kwargs):
    return Model()


_state = {"n": 0, "ev0": None}


def train_step(*, model, extern_data, **_kwargs):
    _bc._ref_hook(_state, _W, _K, _frames, {"metric": "train seconds-of-audio per second", "unit": "audio-s/s", "model": "conformer-aed 12x512 + 6-layer decoder, CE(ls 0.1) + 0.3 CTC (reference rf modules)", "count_scale": 0.01, "parallelism": _parallelism})
    data, targets = extern_data["data"], extern_data["classes"]
    enc, enc_spatial = model.encoder(data, in_spatial_dim=time_dim)
    ctc = rf.ctc_loss(logits=model.aux_ctc(enc), targets=targets, input_spatial_dim=enc_spatial, targets_spatial_dim=targets_time, blank_index=10000)
    ctc.mark_as_loss("ctc", scale=0.3, custom_inv_norm_factor=targets_time.get_size_tensor(), use_normalized_loss=False)
    inp, (tgt_ext,) = rf.pad(targets, axes=[targets_time], padding=[(1, 0)], value=0)
    out_t, _ = rf.pad(targets, axes=[targets_time], padding=[(0, 1)], value=0, out_dims=[tgt_ext], handle_dynamic_dims=True)
    enc_state = model.decoder.transform_encoder(enc, axis=enc_spatial)
    logits, _ = model.decoder(inp, spatial_dim=tgt_ext, encoder=enc_state, state=model.decoder.default_initial_state(batch_dims=[batch_dim]))
    log_prob = rf.log_softmax(logits, axis=vocab_dim)
    log_prob = rf.label_smoothed_log_prob_gradient(log_prob, 0.1, axis=vocab_dim)
    ce = rf.cross_entropy(target=out_t, estimated=log_prob, estimated_type="log-probs", axis=vocab_dim)
    ce.mark_as_loss("ce", use_normalized_loss=True)
    err = rf.reduce_argmax(logits, axis=vocab_dim) != out_t
    err.mark_as_loss("fer", as_error=True)
'''


_REF_BLSTM_CONFIG = r'''#!rnn.py
import os, sys, time, json
import numpy, torch
from returnn.tensor import Tensor, Dim, batch_dim, TensorDict
import returnn.frontend as rf

_opts = __OPTS__
sys.path.insert(0, _opts["root"])
import bench_configs as _bc

backend = "torch"
task = "train"
behavior_version = 24
_W, _K = _opts["warmup"], _opts["steps"]
_rank, _world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
_batches = _bc._asr_batches(4321 + _rank, _W + _K + 1, 20000, 500, 1600, (0.1, 0.25))
_parallelism = "dp%i" % _world
if _world > 1:
    torch_distributed = {"reduce_type": "grad"}
_frames = [sum(s["data"].shape[0] for s in b) for b in _batches]
train = {"class": "StaticDataset", "data": [s for b in _batches for s in b], "output_dim": {"data": (80, 2), "classes": (10000, 1)}}
time_dim = Dim(None, name="time", kind=Dim.Types.Spatial)
feat_dim = Dim(80, name="feature", kind=Dim.Types.Feature)
targets_time = Dim(None, name="targets-time", kind=Dim.Types.Spatial)
vocab_dim = Dim(10000, name="vocab", kind=Dim.Types.Feature)
extern_data = {
    "data": {"dims": (batch_dim, time_dim, feat_dim), "dtype": "float32"},
    "classes": {"dims": (batch_dim, targets_time), "sparse_dim": vocab_dim, "dtype": "int32", "available_for_inference": False},
}
batch_size = 20000
max_seqs = 2000
batching = "default"
optimizer = {"class": "adamw", "weight_decay": 0.01}
learning_rate = 1e-4
torch_amp = "bfloat16"
num_epochs = 1
log_verbosity = 3
torch_dataloader_opts = {"num_workers": 0}


class Blstm(rf.Module):
    def __init__(self, in_dim, hidden):
        super().__init__()
        self.fw = rf.LSTM(in_dim, hidden)
        self.bw = rf.LSTM(in_dim, hidden)
        self.out_dim = hidden + hidden

    def __call__(self, x, *, spatial_dim):
        yf, _ = self.fw(x, state=self.fw.default_initial_state(batch_dims=[batch_dim]), spatial_dim=spatial_dim)
        xr = rf.reverse_sequence(x, axis=spatial_dim)
        yb, _ = self.bw(xr, state=self.bw.default_initial_state(batch_dims=[batch_dim]), spatial_dim=spatial_dim)
        yb = rf.reverse_sequence(yb, axis=spatial_dim)
        out, _ = rf.concat((yf, self.fw.out_dim), (yb, self.bw.out_dim), out_dim=self.out_dim)
        return out


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        layers, cur = [], feat_dim
        for i in range(6):
            layer = Blstm(cur, Dim(1024, name="lstm%i" % i))
            layers.append(layer)
            cur = layer.out_dim
        self.layers = rf.ModuleList(*layers)
        self.wb = vocab_dim + 1
        self.output = rf.Linear(cur, self.wb)

    def __call__(self, x, *, in_spatial_dim):
        spatial = in_spatial_dim
        for i, layer in enumerate(self.layers):
            x = layer(x, spatial_dim=spatial)
            if i in (0, 1):
                x, spatial = rf.max_pool1d(x, pool_size=2, padding="same", in_spatial_dim=spatial)
        return self.output(x), spatial


def get_model(**_kwargs):
    return Model()


_state = {"n": 0, "ev0": None}


def train_step(*, model, extern_data, **_kwargs):
    _bc._ref_hook(_state, _W, _K, _frames, {"metric": "train seconds-of-audio per second", "unit": "audio-s/s", "model": "blstm-ctc 6x1024 (reference rf.LSTM -> torch.lstm / cuDNN)", "count_scale": 0.01, "parallelism": _parallelism})
    logits, enc_spatial = model(extern_data["data"], in_spatial_dim=time_dim)
    loss = rf.ctc_loss(logits=logits, targets=extern_data["classes"], input_spatial_dim=enc_spatial, targets_spatial_dim=targets_time, blank_index=10000)
    loss.mark_as_loss("ctc", custom_inv_norm_factor=targets_time.get_size_tensor(), use_normalized_loss=False)
'''


def run_blstm_reference(args, config_text: str = None, tag: str = "blstm"):
    """BLSTM-CTC (or ``config_text``) through the unmodified reference on one GPU (its LSTM is torch.lstm, i.e. cuDNN)"""
    import tempfile

    ref_dir = os.path.join(_ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "returnn")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/returnn not installed"}))
        return
    opts = {"root": _ROOT, "warmup": args.warmup, "steps": args.steps}
    tmpdir = tempfile.mkdtemp(prefix="bench_ref_%s_" % tag)
    cfg_path = os.path.join(tmpdir, "%s.ref.config" % tag)
    with open(cfg_path, "w") as f:
        f.write((config_text or _REF_BLSTM_CONFIG).replace("__OPTS__", repr(opts)))
    sys.path.insert(0, ref_dir)
    try:
        import tree  # noqa: F401
    except ImportError:
        sys.path.append(os.path.join(_ROOT, "baseline", "deps"))
    from returnn.__main__ import main as ref_main

    old_stdout = sys.stdout
    try:
        sys.stdout = sys.stderr
        ref_main(["rnn.py", cfg_path])
    except SystemExit:
        pass
    except Exception as exc:
        sys.stdout = old_stdout
        print(json.dumps({"impl": "reference", "unavailable": "the reference run failed: %s: %s" % (type(exc).__name__, str(exc)[:300])}))
    finally:
        sys.stdout = old_stdout


def run_12ax_reference(args):
    """the same task through the unmodified reference (its own engine, datasets and rf backend), when it is installed"""
    import tempfile

    ref_dir = os.path.join(_ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "returnn")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/returnn not installed"}))
        return
    import torch

    torch.set_num_threads(int(os.environ.get("OMP_NUM_THREADS", "8")))
    tmpdir = tempfile.mkdtemp(prefix="bench_ref_12ax_")
    cfg_path = os.path.join(tmpdir, "12ax.ref.config")
    with open(cfg_path, "w") as f:
        f.write(_REF_12AX_CONFIG)
    sys.path.insert(0, ref_dir)
    try:
        import tree  # noqa: F401
    except ImportError:
        sys.path.append(os.path.join(_ROOT, "baseline", "deps"))
    from returnn.__main__ import main as ref_main

    old_stdout = sys.stdout
    t0 = time.perf_counter()
    try:
        sys.stdout = sys.stderr
        ref_main(["rnn.py", cfg_path])
    except SystemExit:
        pass
    finally:
        sys.stdout = old_stdout
    wall = time.perf_counter() - t0
    print(json.dumps({"metric": "12AX 2xBLSTM(100) CPU fp32: wall seconds for 2 epochs x 1000 seqs (incl. start-up)", "value": wall, "unit": "s",
                      "higher_is_better": False, "impl": "reference", "dtype": "fp32", "threads": torch.get_num_threads()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["blstm_ctc", "conformer_aed", "transformer_mt", "12ax"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--task", default="train", choices=["train", "search"], help="search: beam search decoding (conformer_aed, transformer_mt)")
    ap.add_argument("--graph-decoder", action="store_true", help="conformer_aed: decoder and cross entropy as a captured CUDA-graph pair inside the eager step")
    ap.add_argument("--cuda-graph", action="store_true", help="train through the captured whole-step CUDA graph (config option torch_cuda_graph)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"], help="reference: every --config here has a reference arm")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.config == "12ax":
            run_12ax_reference(args)
        elif args.config == "transformer_mt":
            run_blstm_reference(args, config_text=_REF_MT_CONFIG, tag="mt")
        elif args.config == "conformer_aed":
            run_blstm_reference(args, config_text=_REF_AED_CONFIG, tag="aed")
        else:
            run_blstm_reference(args)
    elif args.config == "12ax":
        run_12ax(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
