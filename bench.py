#!/usr/bin/env python3
"""
Benchmark of the flagship training step: Conformer-CTC (12 x 512, 8 heads rel-pos MHSA, FFN 2048, conv kernel 32,
conv2d subsampling x6, CTC over 10k BPE + blank), bf16 compute, AdamW with global-norm clipping at 5, data parallel
over N GPUs of one node, 40k padded frames per GPU and step. Metric: seconds of audio per second of training
(sum of the real input frames x 10 ms / step time), whole job.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same model, data and batches

Data: synthetic, identical for both arms (seeded numpy): 80-dim features ~N(0,1), lengths uniform 300..2000 frames,
labels uniform over 1..9999 with length ~frames/30, greedy in-order batches under the padded-frames budget.

Own arm: ``value`` is device-timed (CUDA events around K steps whose inputs are already on the device, max over ranks);
``e2e`` times the same K steps through ``Engine.run_train_step`` including the host-to-device copy of each batch from
pinned memory and the device-to-host read of the loss (pipelined by the engine: ``stage_batch`` starts the copy of the next
batch on a copy stream, ``read_losses="deferred"`` reads the loss of a step after the next step was issued).
Reference arm: the reference engine's own ``train()`` loop; the timestamps are taken inside the config's ``train_step``
hook at the start of step W and the start of step W+K (device synchronised), which brackets exactly K full steps.
"""

from __future__ import annotations
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

_ROOT = os.path.dirname(os.path.abspath(__file__))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

FRAME_SEC = 0.01
MODEL_OPTS = dict(num_layers=12, model_dim=512, num_heads=8, ff_dim=2048, conv_kernel_size=32, in_dim=80, vocab=10000,
                  dropout=0.1, att_dropout=0.1, conv_channels=(32, 64, 64))
BATCH_FRAMES = 40000
BASELINE_PUBLISHED = None  # the reference publishes no number for this config


def make_synth_batches(*, seed: int, n_steps: int, frames_budget: int = BATCH_FRAMES, min_len: int = 300, max_len: int = 2000,
                       feat_dim: int = 80, vocab: int = 10000, shape_seed: int = 1234):
    """
    list of batches; a batch is a list of {"data": [T,F] float32, "classes": [S] int32}.
    The sequence lengths come from ``shape_seed`` (the same on every rank: in a weak-scaling run all ranks then do the same
    amount of work per step and the step time is not the maximum over differently sized random batches), the values from ``seed``.
    """
    import numpy

    rng = numpy.random.RandomState(seed)
    rng_len = numpy.random.RandomState(shape_seed)
    batches, cur, cur_max = [], [], 0
    while len(batches) < n_steps:
        t = int(rng_len.randint(min_len, max_len + 1))
        s = max(1, int(round(t / 30.0)))
        seq = {"data": rng.standard_normal((t, feat_dim)).astype("float32"),
               "classes": rng.randint(1, vocab, size=(s,)).astype("int32")}
        new_max = max(cur_max, t)
        if cur and new_max * (len(cur) + 1) > frames_budget:
            batches.append(cur)
            cur, cur_max = [seq], t
        else:
            cur.append(seq)
            cur_max = new_max
    return batches


class ClockSampler:
    """samples SM clock and throttle reasons with nvidia-smi while the timed region runs"""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local_rank


def _collate(batch, pin: bool):
    """list of seq dicts -> raw batch dict like the data loader produces"""
    import numpy
    import torch
    from returnn_b200.torch.data.pipeline import collate_batch

    items = []
    for i, s in enumerate(batch):
        d = dict(s)
        d["seq_tag"] = numpy.array("seq-%i" % i)
        items.append(d)
    raw = collate_batch(items)
    if pin:
        for k, v in list(raw.items()):
            if isinstance(v, torch.Tensor) and k in ("data", "classes"):
                raw[k] = v.pin_memory()
    return raw


def run_ours(args):
    import numpy
    import torch
    import torch.distributed as dist
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.log import log
    from returnn_b200.utils.basic import BehaviorVersion
    from returnn_b200.models import conformer_ctc
    from returnn_b200.torch.engine import Engine
    from returnn_b200.datasets.generating import StaticDataset
    from returnn_b200.ops import _lib

    rank, world, local_rank = _dist_env()
    assert world == args.gpus, "WORLD_SIZE %i != --gpus %i (launch with torchrun for N>1)" % (world, args.gpus)
    tiny = os.environ.get("BENCH_TINY") == "1"
    if not torch.cuda.is_available() and not tiny:
        raise SystemExit("bench.py needs a GPU")
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank)
    W, K = args.warmup, args.steps
    n_steps = W + K
    # weak scaling: every rank gets its own 40k-frame batches
    batches = make_synth_batches(seed=1234 + rank, n_steps=2 * n_steps, frames_budget=BATCH_FRAMES)
    extern_data = conformer_ctc.make_extern_data(MODEL_OPTS)
    cfg = Config({
        "task": "train", "backend": "torch", "behavior_version": 21, "extern_data": extern_data, "model_opts": dict(MODEL_OPTS),
        "get_model": conformer_ctc.get_model, "train_step": conformer_ctc.train_step,
        "batch_size": BATCH_FRAMES, "max_seqs": 200, "optimizer": {"class": "adamw", "weight_decay": 0.01, "eps": 1e-8},
        "learning_rate": 1e-4, "gradient_clip_global_norm": 5.0, "torch_amp": "bfloat16", "num_epochs": 1,
        "log_verbosity": 2 if rank == 0 else 1, "device": "cuda" if use_cuda else "cpu",
    })
    if world > 1:
        cfg.set("torch_distributed", {"reduce_type": "grad"})
    set_global_config(cfg)
    BehaviorVersion._reset(21)
    log.init_by_config(cfg)
    flat = [s for b in batches[:2] for s in b]
    train_data = StaticDataset(data=flat, output_dim={"data": (80, 2), "classes": (10000, 1)})
    train_data.initialize()
    engine = Engine(cfg)
    engine.init_train_from_config(cfg, train_data, None, None)
    engine.epoch = 1
    engine._pt_model.train()
    dev = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    if not use_cuda:
        _cpu_smoke(engine, batches, W, K)
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    raws = [_collate(b, pin=True) for b in batches]
    frames_per_step = [int(r["data:seq_len"].sum()) for r in raws]

    def to_dev(raw):
        out = dict(raw)
        for k in ("data", "classes"):
            out[k] = raw[k].to(dev, non_blocking=True)
        return out

    # ---- device-timed: inputs staged on the device before the timed region
    for i in range(W):
        engine.run_train_step(to_dev(raws[i]), read_losses=False)
    staged = [to_dev(raws[W + i]) for i in range(K)]
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(K):
        engine.run_train_step(staged[i], read_losses=False)
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = _lib.launch_count() - launches0
    del staged
    # ---- end to end: pinned host -> device every step, loss read back every step.
    # The engine's pipelined form: the copy of batch i+1 is started on the copy stream while step i runs, and the loss of step
    # i is read on the host after step i+1 was issued (the last one by flush_losses), so every step's inputs cross the bus
    # and every step's loss reaches the host inside the timed region, without draining the device queue in between.
    base = n_steps
    staged = engine.stage_batch(raws[base])
    for i in range(min(W, 3)):  # warm-up through the same pipelined path (copy stream, pinned loss ring)
        nxt = engine.stage_batch(raws[base + i + 1]) if i + 1 < min(W, 3) else None
        engine.run_train_step(staged, read_losses="deferred")
        staged = nxt
    engine.flush_losses()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h2d = d2h = 0
    last_loss = None
    n_read = 0
    first = base + min(W, 3)
    staged = engine.stage_batch(raws[first])
    for i in range(K):
        raw = raws[first + i]
        h2d += raw["data"].numel() * raw["data"].element_size() + raw["classes"].numel() * raw["classes"].element_size()
        nxt = engine.stage_batch(raws[first + i + 1]) if i + 1 < K else None
        losses = engine.run_train_step(staged, read_losses="deferred")
        staged = nxt
        if losses:
            n_read += 1
            d2h += 4 * len(losses)
            last_loss = losses
    losses = engine.flush_losses()
    n_read += 1
    d2h += 4 * max(len(losses), 1)
    last_loss = losses
    e1.record()
    barrier()
    assert n_read == K, "every step's loss must have been read on the host (%i of %i)" % (n_read, K)
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if getattr(args, "profile_ops", False) and rank == 0:
        # outside every timed region: per-op times of the native encoder calls (warm caches, events between the ops)
        from returnn_b200.models import conformer_native

        # host issue time: how long the host needs to enqueue K steps (no synchronisation inside); close to the device time
        # means the step is bound by the launching thread, not by the kernels
        torch.cuda.synchronize()
        th0 = time.perf_counter()
        for i in range(K):
            engine.run_train_step(raws[base + i], read_losses=False)
        th1 = time.perf_counter()
        torch.cuda.synchronize()
        th2 = time.perf_counter()
        print("host issue %.3f ms/step, until the device is done %.3f ms/step" % ((th1 - th0) * 1e3 / K, (th2 - th0) * 1e3 / K), file=sys.stderr)
        conformer_native.profile_ops(True)
        for i in range(K):
            engine.run_train_step(raws[base + i], read_losses=False)
        torch.cuda.synchronize()
        rep = conformer_native.profile_report()
        conformer_native.profile_ops(False)
        total = sum(v[1] for v in rep.values()) or 1.0
        host_total = sum(v[2] for v in rep.values())
        print("op profile over %i steps (encoder executor only): device %.3f ms/step, host issue %.3f ms/step" % (K, total / K, host_total / K), file=sys.stderr)
        for tag, (cnt, ms, host) in sorted(rep.items(), key=lambda kv: -kv[1][1]):
            print("  %-22s %6i calls  %9.3f ms/step  %7.1f us/call  %5.1f %%   host %6.1f us/call" % (
                tag, cnt // K, ms / K, 1e3 * ms / max(cnt, 1), 100.0 * ms / total, 1e3 * host / max(cnt, 1)), file=sys.stderr)
    frames_dev = sum(frames_per_step[W: W + K])
    frames_e2e = sum(frames_per_step[base + min(W, 3): base + min(W, 3) + K])
    # max time over ranks, total frames over ranks
    t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
    f = torch.tensor([frames_dev, frames_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
    dev_ms, e2e_ms = t.tolist()
    frames_dev, frames_e2e = f.tolist()
    if rank == 0:
        value = frames_dev * FRAME_SEC / (dev_ms / 1e3)
        e2e_value = frames_e2e * FRAME_SEC / (e2e_ms / 1e3)
        out = {
            "metric": "train seconds-of-audio per second", "value": value, "unit": "audio-s/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None, "dtype": "bf16", "data": "synthetic",
            "impl": "returnn_b200",
            "config": {"model": "conformer-ctc 12x512 h8 ff2048 conv32 sub6 vocab10k", "global_batch": "%i padded frames per GPU x %i" % (BATCH_FRAMES, world),
                       "seq_len": "300-2000 frames (10 ms)", "parallelism": "dp%i" % world, "optimizer": "adamw clip5",
                       "l2": "working set per step (fp32 params, grads, Adam moments ~1.5 GB) exceeds L2; a distinct batch every step",
                       "batches": "sequence lengths drawn from one seed on every rank (equal work per rank), feature and label values per rank",
                       "native_lib": os.path.exists(_lib.lib_path())},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "audio-s/s", "ms_per_step": e2e_ms / K, "h2d_bytes_per_step": h2d // K, "d2h_bytes_per_step": d2h // K,
                    "last_loss": last_loss},
            "gpu_launches": launches,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _cpu_smoke(engine, batches, W, K):
    """--tiny without a GPU: run the steps and print the losses (no timing claims)"""
    t0 = time.perf_counter()
    losses = None
    for i in range(W + K):
        losses = engine.run_train_step(_collate(batches[i], pin=False), read_losses=True)
    print(json.dumps({"impl": "returnn_b200", "tiny_cpu_smoke": True, "steps": W + K, "sec": time.perf_counter() - t0, "last_loss": losses}))


_REF_CONFIG = r'''
import os, sys, time, json
import numpy, torch
from returnn.tensor import Tensor, Dim, batch_dim, TensorDict
import returnn.frontend as rf
from returnn.frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample

_bench = __BENCH_OPTS__
sys.path.insert(0, _bench["root"])
import bench as _bench_mod

backend = "torch"
task = "train"
behavior_version = 21
_rank = int(os.environ.get("RANK", "0"))
_world = int(os.environ.get("WORLD_SIZE", "1"))
_W, _K = _bench["warmup"], _bench["steps"]
_batches = _bench_mod.make_synth_batches(seed=1234 + _rank, n_steps=_W + _K + 1, frames_budget=_bench["batch_frames"])
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
batch_size = _bench["batch_frames"]
max_seqs = 200
batching = "default"
optimizer = {"class": "adamw", "weight_decay": 0.01, "epsilon": 1e-8}
learning_rate = 1e-4
gradient_clip_global_norm = 5.0
torch_amp = "bfloat16"
num_epochs = 1
log_verbosity = 3
torch_dataloader_opts = {"num_workers": 0}  # StaticDataset of the reference does not pickle into a worker process
if _world > 1:
    torch_distributed = {"reduce_type": "grad"}


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        o = _bench["model"]
        self.model_dim = Dim(o["model_dim"], name="enc-model")
        c1, c2, c3 = o["conv_channels"]
        self.encoder = ConformerEncoder(
            feat_dim, self.model_dim, num_layers=o["num_layers"], num_heads=o["num_heads"], ff_dim=Dim(o["ff_dim"], name="enc-ff"),
            conv_kernel_size=o["conv_kernel_size"], dropout=o["dropout"], att_dropout=o["att_dropout"],
            input_layer=ConformerConvSubsample(feat_dim, out_dims=[Dim(c1, name="conv1"), Dim(c2, name="conv2"), Dim(c3, name="conv3")],
                                               filter_sizes=[(3, 3), (3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)]))
        self.wb_vocab_dim = vocab_dim + 1
        self.logits = rf.Linear(self.model_dim, self.wb_vocab_dim)

    def __call__(self, source, *, in_spatial_dim):
        enc, enc_spatial_dim = self.encoder(source, in_spatial_dim=in_spatial_dim)
        return self.logits(enc), enc_spatial_dim


def get_model(*, epoch, step, **_kwargs):
    return Model()


_state = {"n": 0, "t0": None, "ev0": None}


def train_step(*, model, extern_data, **_kwargs):
    n = _state["n"]
    if (n == _W or n == _W + _K) and not torch.cuda.is_available():
        if n == _W:
            _state["t0"] = time.perf_counter()
        else:
            sys.__stdout__.write(json.dumps({"impl": "reference", "tiny_cpu_smoke": True, "sec": time.perf_counter() - _state["t0"]}) + "\n")
    elif n == _W or n == _W + _K:
        torch.cuda.synchronize()
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.barrier()
            torch.cuda.synchronize()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        if n == _W:
            _state["ev0"] = ev
            _state["t0"] = time.perf_counter()
            _bench_mod._ref_timed_region_start(_rank)
        else:
            torch.cuda.synchronize()
            ms = _state["ev0"].elapsed_time(ev)
            _bench_mod._ref_timed_region_end(_rank, _world, ms, sum(_frames[_W:_W + _K]), _W, _K)
    _state["n"] = n + 1
    data = extern_data["data"]
    targets = extern_data["classes"]
    logits, enc_spatial_dim = model(data, in_spatial_dim=time_dim)
    loss = rf.ctc_loss(logits=logits, targets=targets, input_spatial_dim=enc_spatial_dim, targets_spatial_dim=targets_time, blank_index=10000)
    loss.mark_as_loss("ctc", custom_inv_norm_factor=targets_time.get_size_tensor(), use_normalized_loss=False)
'''

_ref_sampler = None


def _ref_timed_region_start(rank: int):
    global _ref_sampler
    if rank == 0:
        _ref_sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
        _ref_sampler.start()


def _ref_timed_region_end(rank: int, world: int, ms: float, frames: int, W: int, K: int):
    import torch
    import torch.distributed as dist

    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    f = torch.tensor([float(frames)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
    if rank == 0:
        clocks = _ref_sampler.stop() if _ref_sampler else None
        ms_, frames_ = t.item(), f.item()
        value = frames_ * FRAME_SEC / (ms_ / 1e3)
        out = {"impl": "reference", "metric": "train seconds-of-audio per second", "value": value, "unit": "audio-s/s", "n_gpus": world,
               "steps": K, "warmup": W, "ms_per_step": ms_ / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
               "dtype": "bf16", "data": "synthetic",
               "config": {"model": "conformer-ctc 12x512 h8 ff2048 conv32 sub6 vocab10k", "global_batch": "%i padded frames per GPU x %i" % (BATCH_FRAMES, world),
                          "seq_len": "300-2000 frames (10 ms)", "parallelism": "dp%i" % world, "optimizer": "adamw clip5",
                          "timing": "engine train() loop, timestamps in train_step at steps W and W+K (end to end incl. data loading, H2D, loss .item())"},
               "clocks": clocks, "e2e": {"value": value, "unit": "audio-s/s", "note": "the reference number is end to end by construction"}}
        sys.__stdout__.write(json.dumps(out) + "\n")
        sys.__stdout__.flush()


def run_reference(args):
    ref_dir = os.path.join(_ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "returnn")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/returnn not installed"}))
        return
    try:
        import torch

        if not torch.cuda.is_available() and os.environ.get("BENCH_TINY") != "1":
            print(json.dumps({"impl": "reference", "unavailable": "no GPU visible"}))
            return
    except Exception as exc:
        print(json.dumps({"impl": "reference", "unavailable": "torch import failed: %s" % exc}))
        return
    import tempfile

    rank, world, local_rank = _dist_env()
    opts = {"root": _ROOT, "warmup": args.warmup, "steps": args.steps, "model": dict(MODEL_OPTS), "batch_frames": BATCH_FRAMES}
    cfg_text = "#!rnn.py\n" + _REF_CONFIG.replace("__BENCH_OPTS__", repr(opts))
    tmpdir = tempfile.mkdtemp(prefix="bench_ref_%i_" % rank)
    cfg_path = os.path.join(tmpdir, "conformer_ctc.ref.config")
    with open(cfg_path, "w") as f:
        f.write(cfg_text)
    sys.path.insert(0, ref_dir)
    # the reference imports dm-tree ("import tree"), which this image lacks: a small pure-Python stand-in
    try:
        import tree  # noqa: F401
    except ImportError:
        sys.path.append(os.path.join(_ROOT, "baseline", "deps"))
    try:
        from returnn.__main__ import main as ref_main
    except Exception as exc:
        print(json.dumps({"impl": "reference", "unavailable": "import of the reference failed: %s: %s" % (type(exc).__name__, str(exc)[:200])}))
        return
    old_stdout = sys.stdout
    try:
        # the reference logs to stdout; the JSON line goes to the real stdout, its log to stderr
        sys.stdout = sys.stderr
        ref_main(["rnn.py", cfg_path])
    except SystemExit:
        pass
    except Exception as exc:
        sys.stdout = old_stdout
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference run failed: %s: %s" % (type(exc).__name__, str(exc)[:300])}))
        return
    finally:
        sys.stdout = old_stdout


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-ops", action="store_true", help="after the measurement, print per-op times of the native encoder to stderr")
    ap.add_argument("--tiny", action="store_true", help="small model and batches on any device: a functional smoke test, not a benchmark")
    args = ap.parse_args()
    if args.tiny:
        global BATCH_FRAMES
        MODEL_OPTS.update(num_layers=2, model_dim=64, num_heads=4, ff_dim=128, conv_channels=(4, 8, 8))
        BATCH_FRAMES = 4000
        os.environ["BENCH_TINY"] = "1"
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
