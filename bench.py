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


CONFIG_MODEL = "conformer-ctc 12x512 h8 ff2048 conv32 sub6 vocab10k"


def common_config(world: int):
    """the ``config`` entry of the JSON line: identical in both arms (what is specific to an arm goes to ``notes``)"""
    return {
        "model": CONFIG_MODEL, "global_batch": "%i padded frames per GPU x %i" % (BATCH_FRAMES, world),
        "seq_len": "300-2000 frames (10 ms)", "parallelism": "dp%i" % world, "optimizer": "adamw clip5",
        "l2": "no flush needed: the working set of a step (fp32 parameters, gradients and Adam moments 1.3 GB, saved activations 2.3 GB) is "
              "far larger than the 126 MB L2, and every step gets a distinct batch",
        "batches": "sequence lengths drawn from one seed on every rank (equal work per rank), feature and label values per rank"}


def balanced_rank_batches(*, rank: int, world: int, n_steps: int, frames_budget: int = BATCH_FRAMES):
    """
    Batches of a data-parallel job whose ranks all read the SAME sequence stream: every group of ``world`` consecutive greedy
    batches is re-divided so that the ranks get near-equal real frame totals (``returnn_b200.torch.data.pipeline.balance_batches``,
    what ``torch_batching = {"type": "rank_balanced"}`` does in training); this rank keeps part ``rank`` of every group.
    """
    from returnn_b200.torch.data.pipeline import balance_batches

    stream = make_synth_batches(seed=999, n_steps=n_steps * world, frames_budget=frames_budget, shape_seed=777)
    out = []
    for step in range(n_steps):
        group = stream[step * world: (step + 1) * world]
        out.append(balance_batches(group, length_key="data", max_seqs=200)[rank])
    return out


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
    from returnn_b200.ops import status as status_board

    rank, world, local_rank = _dist_env()
    assert world == args.gpus, "WORLD_SIZE %i != --gpus %i (launch with torchrun for N>1)" % (world, args.gpus)
    tiny = os.environ.get("BENCH_TINY") == "1"
    if not torch.cuda.is_available() and not tiny:
        raise SystemExit("bench.py needs a GPU")
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank)
    W, K = args.warmup, args.steps
    # weak scaling: every rank gets its own 40k-frame batches; W warm-up batches, K timed ones, one more so that step W+K starts
    batches = make_synth_batches(seed=1234 + rank, n_steps=W + K + 1, frames_budget=BATCH_FRAMES)
    extern_data = conformer_ctc.make_extern_data(MODEL_OPTS)
    hook = {"armed": False, "n": 0, "ev0": None, "ev1": None}

    def train_step(*, model, extern_data, **kwargs):
        """the model's train_step; while armed (the Engine.train() measurement) it takes the timestamps at the start of steps W and W+K"""
        if hook["armed"]:
            n = hook["n"]
            if n in (W, W + K) and use_cuda:
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                    torch.cuda.synchronize()
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                hook["ev0" if n == W else "ev1"] = ev
            hook["n"] = n + 1
        return conformer_ctc.train_step(model=model, extern_data=extern_data, **kwargs)

    cfg = Config({
        "task": "train", "backend": "torch", "behavior_version": 24, "extern_data": extern_data, "model_opts": dict(MODEL_OPTS),
        "get_model": conformer_ctc.get_model, "train_step": train_step,
        "batch_size": BATCH_FRAMES, "max_seqs": 200, "optimizer": {"class": "adamw", "weight_decay": 0.01, "eps": 1e-8},
        "learning_rate": 1e-4, "gradient_clip_global_norm": 5.0, "torch_amp": "bfloat16", "num_epochs": 1,
        "log_verbosity": 2 if rank == 0 else 1, "device": "cuda" if use_cuda else "cpu",
    })
    if world > 1:
        cfg.set("torch_distributed", {"reduce_type": "grad"})
    set_global_config(cfg)
    BehaviorVersion._reset(24)
    log.init_by_config(cfg)
    # the dataset of the Engine.train() measurement: the sequences of all batches in order; the engine's greedy batching under the same
    # budget re-creates exactly these batches (the reference arm feeds its engine the same way)
    train_data = StaticDataset(data=[s for b in batches for s in b], output_dim={"data": (80, 2), "classes": (10000, 1)})
    train_data.initialize()
    engine = Engine(cfg)
    engine.init_train_from_config(cfg, train_data, None, None)
    engine.epoch = 1
    engine._pt_model.train()
    dev = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    if not use_cuda:
        _cpu_smoke(engine, batches, W, K)
        return None

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
    status_board.check_now(dev)
    # ---- end to end through run_train_step on the SAME K batches: pinned host -> device every step, loss read back every step.
    # The engine's pipelined form: the copy of batch i+1 is started on the copy stream while step i runs, and the loss of step
    # i is read on the host after step i+1 was issued (the last one by flush_losses), so every step's inputs cross the bus
    # and every step's loss reaches the host inside the timed region, without draining the device queue in between.
    n_warm = min(W, 3)
    staged = engine.stage_batch(raws[0])
    for i in range(n_warm):  # warm-up through the same pipelined path (copy stream, pinned loss ring)
        nxt = engine.stage_batch(raws[i + 1]) if i + 1 < n_warm else None
        engine.run_train_step(staged, read_losses="deferred")
        staged = nxt
    engine.flush_losses()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h2d = d2h = 0
    last_loss = None
    n_read = 0
    staged = engine.stage_batch(raws[W])
    for i in range(K):
        raw = raws[W + i]
        h2d += raw["data"].numel() * raw["data"].element_size() + raw["classes"].numel() * raw["classes"].element_size()
        nxt = engine.stage_batch(raws[W + i + 1]) if i + 1 < K else None
        losses = engine.run_train_step(staged, read_losses="deferred")
        staged = nxt
        if losses:
            n_read += 1
            last_loss = losses
    losses = engine.flush_losses()
    n_read += 1
    last_loss = losses or last_loss
    e1.record()
    barrier()
    assert n_read == K, "every step's loss must have been read on the host (%i of %i)" % (n_read, K)
    d2h = K * (4 * max(len(last_loss or {}), 1) + 4 * status_board.NUM_SLOTS)  # the losses and the kernel status board, every step
    rts_ms = e0.elapsed_time(e1)
    # ---- end to end through Engine.train(): dataset -> batching -> collation -> pinned memory -> device -> step -> loss on the host,
    # the loop a user runs. Timestamps at the start of steps W and W+K inside train_step (device synchronised, ranks aligned), as in
    # the reference arm.
    train_ms = None
    train_err = None
    try:
        hook.update(armed=True, n=0, ev0=None, ev1=None)
        engine.train()
        hook["armed"] = False
        if hook["ev0"] is not None and hook["ev1"] is not None:
            torch.cuda.synchronize()
            train_ms = hook["ev0"].elapsed_time(hook["ev1"])
        else:
            train_err = "the engine ran %i steps, fewer than warm-up + timed steps" % hook["n"]
    except Exception as exc:  # the device-timed number stands on its own; say what happened
        hook["armed"] = False
        train_err = "%s: %s" % (type(exc).__name__, str(exc)[:200])
    clocks = sampler.stop() if rank == 0 else None
    engine._pt_model.train()
    # ---- data parallel only: batches whose shapes differ between the ranks (what real training has), device-timed
    distinct = None
    if world > 1:
        distinct = {}
        n_d = min(K, 20)
        for name, bs in (("independent", make_synth_batches(seed=4321 + rank, n_steps=2 + n_d, shape_seed=5000 + rank)),
                         ("rank_balanced", balanced_rank_batches(rank=rank, world=world, n_steps=2 + n_d))):
            rs = [_collate(b, pin=True) for b in bs]
            for i in range(2):
                engine.run_train_step(to_dev(rs[i]), read_losses=False)
            st = [to_dev(rs[2 + i]) for i in range(n_d)]
            barrier()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(n_d):
                engine.run_train_step(st[i], read_losses=False)
            b_.record()
            barrier()
            tt = torch.tensor([a.elapsed_time(b_)], device=dev, dtype=torch.float64)
            ff = torch.tensor([float(sum(int(r["data:seq_len"].sum()) for r in rs[2:]))], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dist.all_reduce(ff, op=dist.ReduceOp.SUM)
            distinct[name] = {"ms_per_step": tt.item() / n_d, "value": ff.item() * FRAME_SEC / (tt.item() / 1e3), "steps": n_d}
            del st, rs
    status_board.check_now(dev)
    if getattr(args, "profile_ops", False) and rank == 0:
        _profile_ops(engine, raws, W, K)
    frames = sum(frames_per_step[W: W + K])
    # parameters after the same number of steps on every rank: max - min over the ranks of sum |p| (0 = the ranks hold the same model)
    checksum = torch.stack([p.detach().double().abs().sum() for p in engine._pt_model.parameters()]).sum().reshape(1)
    spread = 0.0
    if world > 1:
        allc = [torch.zeros_like(checksum) for _ in range(world)]
        dist.all_gather(allc, checksum)
        allc = torch.cat(allc)
        spread = float(allc.max() - allc.min())
    # max time over ranks, total frames over ranks
    t = torch.tensor([dev_ms, rts_ms, train_ms if train_ms is not None else -1.0], device=dev, dtype=torch.float64)
    f = torch.tensor([frames], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
    dev_ms, rts_ms, train_ms_all = t.tolist()
    frames = f.item()
    dist_ctx = engine._torch_distributed_ctx
    out = None
    if rank == 0:
        value = frames * FRAME_SEC / (dev_ms / 1e3)
        rts = {"value": frames * FRAME_SEC / (rts_ms / 1e3), "ms_per_step": rts_ms / K,
               "api": "Engine.stage_batch + Engine.run_train_step(read_losses='deferred') on pre-collated pinned batches"}
        if train_ms is not None and train_ms_all > 0:
            e2e = {"value": frames * FRAME_SEC / (train_ms_all / 1e3), "unit": "audio-s/s", "ms_per_step": train_ms_all / K,
                   "h2d_bytes_per_step": h2d // K, "d2h_bytes_per_step": d2h // K,
                   "api": "Engine.train(): StaticDataset -> greedy batching -> collation -> pinned memory -> device -> step -> loss on the host, every step",
                   "run_train_step": rts, "last_loss": last_loss}
        else:
            e2e = dict(rts, unit="audio-s/s", h2d_bytes_per_step=h2d // K, d2h_bytes_per_step=d2h // K, last_loss=last_loss,
                       engine_train_error=train_err)
        out = {
            "metric": "train seconds-of-audio per second", "value": value, "unit": "audio-s/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None, "dtype": "bf16", "data": "synthetic",
            "impl": "returnn_b200", "config": common_config(world), "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "grad_reduce": dist_ctx.grad_reduce_mode if dist_ctx else "none", "param_checksum_spread": spread,
            "notes": {"native_lib": os.path.exists(_lib.lib_path()), "value_and_e2e": "the same K batches in all three measurements",
                      "distinct_shapes": distinct},
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


def _profile_ops(engine, raws, W, K):
    """outside every timed region: per-op times of the native encoder calls (warm caches, events between the ops), to stderr"""
    import torch
    from returnn_b200.models import conformer_native

    # host issue time: how long the host needs to enqueue K steps (no synchronisation inside); close to the device time
    # means the step is bound by the launching thread, not by the kernels
    torch.cuda.synchronize()
    th0 = time.perf_counter()
    for i in range(K):
        engine.run_train_step(raws[W + i], read_losses=False)
    th1 = time.perf_counter()
    torch.cuda.synchronize()
    th2 = time.perf_counter()
    print("host issue %.3f ms/step, until the device is done %.3f ms/step" % ((th1 - th0) * 1e3 / K, (th2 - th0) * 1e3 / K), file=sys.stderr)
    conformer_native.profile_ops(True)
    for i in range(K):
        engine.run_train_step(raws[W + i], read_losses=False)
    torch.cuda.synchronize()
    rep = conformer_native.profile_report()
    conformer_native.profile_ops(False)
    total = sum(v[1] for v in rep.values()) or 1.0
    host_total = sum(v[2] for v in rep.values())
    print("op profile over %i steps (encoder executor only): device %.3f ms/step, host issue %.3f ms/step" % (K, total / K, host_total / K), file=sys.stderr)
    for tag, (cnt, ms, host) in sorted(rep.items(), key=lambda kv: -kv[1][1]):
        print("  %-22s %6i calls  %9.3f ms/step  %7.1f us/call  %5.1f %%   host %6.1f us/call" % (
            tag, cnt // K, ms / K, 1e3 * ms / max(cnt, 1), 100.0 * ms / total, 1e3 * host / max(cnt, 1)), file=sys.stderr)


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
behavior_version = 24
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
            conv_norm=rf.build_dict(rf.BatchNorm, use_mask=True),
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
_ref_result = None


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
        global _ref_result
        _ref_result = {"impl": "reference", "metric": "train seconds-of-audio per second", "value": value, "unit": "audio-s/s", "n_gpus": world,
                       "steps": K, "warmup": W, "ms_per_step": ms_ / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                       "dtype": "bf16", "data": "synthetic", "config": common_config(world), "clocks": clocks,
                       "e2e": {"value": value, "unit": "audio-s/s", "ms_per_step": ms_ / K,
                               "note": "the reference number is end to end by construction: its engine's train() loop"},
                       "notes": {"timing": "engine train() loop, timestamps in train_step at steps W and W+K (end to end incl. data loading, "
                                           "H2D, loss .item())"}}


def run_reference(args):
    """:return: the JSON dict of the reference arm (rank 0; ``{"impl": "reference", "unavailable": ...}`` if it cannot run), None on other ranks"""
    ref_dir = os.path.join(_ROOT, "baseline", "_ref")
    rank, world, local_rank = _dist_env()

    def unavailable(why):
        return {"impl": "reference", "unavailable": why}  # on every rank: all of them then skip the secondary runs alike

    if not os.path.isdir(os.path.join(ref_dir, "returnn")):
        return unavailable("baseline/_ref/returnn not installed")
    try:
        import torch

        if not torch.cuda.is_available() and os.environ.get("BENCH_TINY") != "1":
            return unavailable("no GPU visible")
    except Exception as exc:
        return unavailable("torch import failed: %s" % exc)
    import tempfile

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
        return unavailable("import of the reference failed: %s: %s" % (type(exc).__name__, str(exc)[:200]))
    old_stdout = sys.stdout
    try:
        # the reference logs to stdout; the JSON line goes to the real stdout, its log to stderr
        sys.stdout = sys.stderr
        ref_main(["rnn.py", cfg_path])
    except SystemExit:
        pass
    except Exception as exc:
        return unavailable("the reference run failed: %s: %s" % (type(exc).__name__, str(exc)[:300]))
    finally:
        sys.stdout = old_stdout
    # the config imports this file as module "bench" (this script itself runs as __main__): the result was stored there
    mod = sys.modules.get("bench")
    res = getattr(mod, "_ref_result", None) if mod is not None else None
    if res is None and rank == 0:
        return unavailable("the reference engine finished without reaching step warm-up + steps")
    return res if rank == 0 else {}


SECONDARY = ("blstm_ctc", "conformer_aed")


def run_secondary(args, impl: str):
    """
    The other headline configurations, each as a short run of ``bench_configs.py`` in a child process per rank (its own process
    group on another port): BLSTM-CTC (6 x 1024, 20k frames per GPU) and Conformer-AED with parameter averaging
    (``reduce_type="param"``, ``param_sync_step=100``; on more than one GPU the timed region holds 100 steps, so that exactly one
    parameter synchronisation falls into it). A failure or a timeout of a child is reported in its entry; the flagship line stands.

    :return: {name: JSON dict of the child} on rank 0, None on other ranks
    """
    rank, world, local_rank = _dist_env()
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    results = {}
    for idx, name in enumerate(SECONDARY):
        steps = min(args.steps, 10)
        if name == "conformer_aed" and world > 1:
            steps = 100
        cmd = [sys.executable, os.path.join(_ROOT, "bench_configs.py"), "--config", name, "--gpus", str(world), "--steps", str(steps), "--warmup", "3",
               "--impl", impl]
        if name == "conformer_aed" and impl == "ours":
            cmd.append("--graph-decoder")  # decoder + loss as a captured graph pair inside the eager step (models/graphed_decoder.py)
        env = dict(os.environ, MASTER_PORT=str(base_port + 1 + idx), MASTER_ADDR=os.environ.get("MASTER_ADDR", "127.0.0.1"))
        # torchrun's own bookkeeping variables must not reach the child: it forms a process group of its own
        for k in list(env):
            # (the reference engine exports its process-group state to child processes through an environment variable of its own)
            if k.startswith("TORCHELASTIC_") or k.startswith("_RETURNN_") or k in ("GROUP_RANK", "ROLE_RANK", "ROLE_NAME", "GROUP_WORLD_SIZE",
                                                                                   "ROLE_WORLD_SIZE"):
                env.pop(k)
        try:
            p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
            line = None
            for ln in p.stdout.splitlines():
                if ln.startswith("{"):
                    line = ln
            if line is not None:
                results[name] = json.loads(line)
            elif rank == 0:
                results[name] = {"error": "exit code %i, no result line: %s" % (p.returncode, (p.stderr or "")[-300:])}
        except subprocess.TimeoutExpired:
            results[name] = {"error": "timed out after 900 s"}
        except Exception as exc:
            results[name] = {"error": "%s: %s" % (type(exc).__name__, str(exc)[:200])}
    return results if rank == 0 else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-ops", action="store_true", help="after the measurement, print per-op times of the native encoder to stderr")
    ap.add_argument("--tiny", action="store_true", help="small model and batches on any device: a functional smoke test, not a benchmark")
    ap.add_argument("--no-secondary", action="store_true", help="only the flagship configuration (no BLSTM-CTC / Conformer-AED runs afterwards)")
    args = ap.parse_args()
    if args.tiny:
        global BATCH_FRAMES
        MODEL_OPTS.update(num_layers=2, model_dim=64, num_heads=4, ff_dim=128, conv_channels=(4, 8, 8))
        BATCH_FRAMES = 4000
        os.environ["BENCH_TINY"] = "1"
    if args.warmup < 3:
        args.warmup = 3
    rank = _dist_env()[0]
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    have_gpu = False
    try:
        import torch

        have_gpu = torch.cuda.is_available()
        if have_gpu:
            torch.cuda.empty_cache()  # the children of the secondary runs get the device memory
    except Exception:
        pass
    if out is None:
        out = {}  # ranks other than 0 (they take part in the children's process groups below), or the CPU smoke run
    if "unavailable" not in out and have_gpu and not args.tiny and not args.no_secondary:
        sec = run_secondary(args, args.impl)
        if sec is not None:
            out["secondary"] = sec
    if rank == 0 and out:
        sys.__stdout__.write(json.dumps(out) + "\n")
        sys.__stdout__.flush()


if __name__ == "__main__":
    main()
