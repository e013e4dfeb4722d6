"""
The NVLink kernels on two real GPUs (one process per GPU, child processes of the test; skipped with fewer than 2 GPUs):

* the fused gradient all-reduce against an fp64 sum, for ragged sizes (``n % 4 != 0``, fewer than ``4 * world`` elements,
  buckets that start at odd multiples of 4), through plain peer loads and through the NVSwitch multicast mapping;
* the small-vector all-reduce (batch-norm statistics);
* the fused AdamW + parameter averaging against torch ops + ``all_reduce``, while a second stream keeps the SMs busy, so that
  the CTAs of the kernel are not all resident at once;
* three training steps with ``fused: True`` and with ``fused: False`` (NCCL): same parameters;
* a bounded wait that runs out: rank 1 leaves out one launch on the host, rank 0's kernel gives up after 50 ms, writes its
  status word, the host raises ``KernelWaitTimeout``, and the context and the next reduction still work. No GPU faults or
  hangs: the wait is bounded, NVLS is off and the kernel uses plain peer loads.
"""

import os
import socket
import subprocess
import sys
import textwrap
import pytest
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


_HEAD = """
import os, sys, time
sys.path.insert(0, %r)
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("cpu:gloo,cuda:nccl", device_id=dev)
from returnn_b200.parallel.arena import ParamArena
from returnn_b200.parallel import fused_allreduce
from returnn_b200.ops import status as status_board

def host_barrier():
    torch.cuda.synchronize()
    dist.all_reduce(torch.zeros(1))   # a CPU tensor: gloo, nothing on the GPU

def finish(ok=True):
    host_barrier()
    print("RANK_DONE %%i %%s" %% (rank, "OK" if ok else "FAILED"))
    sys.stdout.flush()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)
""" % _ROOT


def _run(body: str, tmp_path, *, world: int = 2, timeout: int = 420, env_extra=None):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(_HEAD) + textwrap.dedent(body))
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        env.update(env_extra or {})
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()  # the exact child this test started
            out, _ = p.communicate()
            out += "\n<killed by the test after %i s>" % timeout
        outs.append((p.returncode, out))
    for r, (rc, out) in enumerate(outs):
        assert rc == 0 and ("RANK_DONE %i OK" % r) in out, "rank %i:\n%s" % (r, out[-4000:])
    return outs


@pytest.mark.parametrize("multimem", ["0", "1"])
def test_fused_allreduce_values_ragged(tmp_path, multimem):
    _run("""
    os.environ["RETURNN_B200_ALLREDUCE_MULTIMEM"] = %r
    # parameter sizes chosen so that buckets start at odd multiples of 4 and have n %% 4 != 0 or n < 4 * world
    sizes = [3, 5, 131, 1, 4099, 7, 100003, 2, 65536 + 1, 6]
    params = [("p%%i" %% i, torch.nn.Parameter(torch.zeros(s, device=dev))) for i, s in enumerate(sizes)]
    arena = ParamArena(params, bucket_bytes=1)   # one bucket per parameter
    red = fused_allreduce.FusedAllReduce(arena, rank=rank, world=world)
    if %r == "1" and not red.multicast_ptr:
        print("no multicast mapping on this machine: peer path tested instead")
    g = arena.flat_grad
    ok = True
    for trial in range(3):
        gen = torch.Generator(device=dev); gen.manual_seed(17 * trial + rank)
        mine = torch.randn(arena.total, device=dev, generator=gen)
        alls = []
        for r in range(world):
            gen_r = torch.Generator(device=dev); gen_r.manual_seed(17 * trial + r)
            alls.append(torch.randn(arena.total, device=dev, generator=gen_r).double())
        want = sum(alls) / world
        g.copy_(mine)
        host_barrier()
        # whole buckets, then ragged sub-ranges: lengths with n %% 4 in {1, 2, 3}, n < 4 * world, starts at odd multiples of 4
        ranges = list(arena.buckets) + [(4, 4 + 5), (12, 12 + 3), (20, 20 + 1), (128 * 3 + 4, 128 * 3 + 4 + 4 * world - 1)]
        covered = torch.zeros(arena.total, dtype=torch.bool, device=dev)
        for b, (lo, hi) in enumerate(arena.buckets):
            red.reduce_bucket(b, lo, hi)
            covered[lo:hi] = True
        norm_sq = red.finish()
        torch.cuda.synchronize()
        red.check_status()
        err = float((g.double() - want)[covered].abs().max())
        ref_norm = float((want[covered] ** 2).sum())
        nerr = abs(float(norm_sq) - ref_norm) / ref_norm
        if err > 1e-6 or nerr > 1e-5:
            print("trial", trial, "max abs err", err, "norm rel err", nerr); ok = False
        # the squared norm is bitwise the same on every rank (it scales the update: a difference in the last bit lets the ranks drift)
        both = [torch.zeros_like(norm_sq.reshape(1)) for _ in range(world)]
        dist.all_gather(both, norm_sq.reshape(1).contiguous())
        if not all(torch.equal(both[0], b) for b in both):
            print("trial", trial, "norm differs between ranks", [float(b) for b in both]); ok = False
        # the ragged sub-ranges on fresh data (every element of the range must be the average, everything else untouched)
        for (lo, hi) in ranges[len(arena.buckets):]:
            g.copy_(mine)
            host_barrier()
            red.reduce_bucket(0, lo, hi)
            red.finish()
            torch.cuda.synchronize()
            red.check_status()
            got = g.double()
            e_in = float((got[lo:hi] - want[lo:hi]).abs().max())
            untouched = torch.ones(arena.total, dtype=torch.bool, device=dev); untouched[lo:hi] = False
            e_out = float((got[untouched] - mine.double()[untouched]).abs().max())
            if e_in > 1e-6 or e_out != 0.0:
                print("range", lo, hi, "err inside", e_in, "outside", e_out); ok = False
    # small-vector all-reduce
    small = fused_allreduce.SmallVectorAllReduce(device=dev, rank=rank, world=world)
    for n in (1, 3, 1025):
        vec = torch.arange(n, device=dev, dtype=torch.float32) * (rank + 1) + 0.5
        got = small.all_reduce_sum(vec)
        want_v = sum(torch.arange(n, device=dev, dtype=torch.float32) * (r + 1) + 0.5 for r in range(world))
        if not torch.equal(got, want_v):
            print("small vector", n, float((got - want_v).abs().max())); ok = False
    status_board.check_now(dev)
    finish(ok)
    """ % (multimem, multimem), tmp_path)


@pytest.mark.parametrize("multimem", ["0", "1"])
def test_fused_adamw_param_avg_with_busy_sms(tmp_path, multimem):
    _run("""
    os.environ["RETURNN_B200_ALLREDUCE_MULTIMEM"] = %r
    from returnn_b200.torch.optim.fused_adamw import FusedArenaAdamW
    torch.manual_seed(0)
    n = 6_000_000
    module = torch.nn.Module()
    module.ps = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(n // 2 + 7, device=dev) * 0.1), torch.nn.Parameter(torch.randn(n // 2, device=dev) * 0.1)])
    opt = FusedArenaAdamW(module, lr=1e-2, weight_decay=0.01)
    arena = opt.arena
    avg = fused_allreduce.FusedParamAverager(arena, rank=rank, world=world)
    opt.param_averager = avg
    start = arena.flat_param.clone()
    gen = torch.Generator(device=dev); gen.manual_seed(100 + rank)
    grads = torch.randn(arena.total, device=dev, generator=gen)
    b1, b2, eps, lr, wd = 0.9, 0.999, 1e-8, 1e-2, 0.01
    m = (1 - b1) * grads
    v = (1 - b2) * grads * grads
    mask = opt.wd_flags.repeat_interleave(128)[: arena.total].float()
    ref = start * (1 - lr * wd * mask) - lr * (m / (1 - b1)) / ((v / (1 - b2)).sqrt() + eps)
    dist.all_reduce(ref)
    ref /= world
    busy = torch.cuda.Stream()
    a = torch.randn(4096, 4096, device=dev)
    ok = True
    for trial in range(4):
        arena.flat_param.copy_(start)
        arena.flat_grad.copy_(grads)
        opt.exp_avg.zero_(); opt.exp_avg_sq.zero_(); opt.step_count = 0
        host_barrier()
        with torch.cuda.stream(busy):
            for _ in range(20 + 10 * rank):   # different load per rank: the CTAs of the two ranks do not run in lock step
                a2 = a @ a
        avg.pending = True
        opt.step()
        torch.cuda.synchronize()
        avg.check_status()
        err = float((arena.flat_param - ref).abs().max())
        if err > 1e-6:
            print("trial", trial, "max abs err", err); ok = False
    finish(ok)
    """ % multimem, tmp_path)


def test_training_steps_fused_equals_nccl(tmp_path):
    _run("""
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.torch import distributed as rdist
    from returnn_b200.torch.updater import Updater

    def train(fused):
        rdist.reset_ctx()
        cfg = Config({"torch_distributed": {"reduce_type": "grad", "fused": fused, "bucket_cap_mb": 1}, "log_verbosity": 3,
                      "optimizer": {"class": "adamw", "weight_decay": 0.01}, "learning_rate": 1e-3, "gradient_clip_global_norm": 1.0})
        set_global_config(cfg)
        ctx = rdist.get_ctx(cfg)
        torch.manual_seed(0)
        net = torch.nn.Sequential(torch.nn.Linear(512, 1024), torch.nn.Tanh(), torch.nn.Linear(1024, 1024), torch.nn.Tanh(), torch.nn.Linear(1024, 8)).to(dev)
        ctx.setup_grad_reduction(net)
        assert (ctx.fused is not None) == bool(fused), (fused, ctx.fused)
        upd = Updater(config=cfg, network=net, device=dev, initial_learning_rate=1e-3)
        upd.set_arena(ctx.arena)
        upd.create_optimizer()
        for step in range(3):
            upd.zero_grad()
            gen = torch.Generator(device=dev); gen.manual_seed(1000 * step + rank)
            x = torch.randn(64, 512, device=dev, generator=gen)
            ctx.prepare_backward(sync=True)
            net(x).square().mean().backward()
            norm_sq = ctx.maybe_reduce_grads(net)
            if norm_sq is not None:
                upd.set_precomputed_grad_norm_sq(norm_sq)
            upd.step()
        torch.cuda.synchronize()
        status_board.check_now(dev)
        return torch.cat([p.detach().reshape(-1) for p in net.parameters()]).clone(), ctx

    p_fused, ctx_f = train(True)
    mode = ctx_f.grad_reduce_mode
    p_nccl, ctx_n = train(False)
    assert ctx_n.grad_reduce_mode == "nccl", ctx_n.grad_reduce_mode
    err = float((p_fused - p_nccl).abs().max())
    # both ranks hold the same parameters
    other = p_fused.clone()
    dist.broadcast(other, src=0)
    spread = float((other - p_fused).abs().max())
    print("mode", mode, "fused vs nccl max abs diff", err, "rank spread", spread)
    finish(err <= 1e-6 and spread == 0.0 and mode.startswith("fused"))
    """, tmp_path)


def test_bounded_wait_runs_out_and_host_raises(tmp_path):
    _run("""
    from returnn_b200.ops.status import KernelWaitTimeout, StatusPoller
    params = [("p0", torch.nn.Parameter(torch.zeros(1 << 20, device=dev)))]
    arena = ParamArena(params)
    red = fused_allreduce.FusedAllReduce(arena, rank=rank, world=world, wait_ms=50)
    assert red.mode == "fused-peer", red.mode
    g = arena.flat_grad
    poller = StatusPoller(dev)

    def step(value):
        g.fill_(value * (rank + 1))
        host_barrier()
        red.reduce_bucket(0, 0, arena.total)
        red.finish()
        poller.step(where="step")

    ok = True
    step(1.0)                                   # a normal step
    torch.cuda.synchronize()
    ok = ok and abs(float(g[0]) - 1.5) < 1e-6
    if rank == 1:
        red.skip_launches = 1                   # the host leaves out rank 1's next launch: rank 0 waits for a flag nothing sets
    raised = None
    try:
        step(2.0)                               # rank 0: the entry barrier runs out after ~50 ms, the kernel returns
        host_barrier()
        step(3.0)                               # the poller looks at the step before this one and raises on rank 0
        poller.flush()
    except KernelWaitTimeout as exc:
        raised = exc
    if rank == 0:
        ok = ok and raised is not None and status_board.SLOT_ALLREDUCE in raised.codes and "peer rank 1" in str(raised)
        print("rank 0 raised:", raised)
    else:
        ok = ok and raised is None
    # the context is usable and the next reductions are correct again (the launch counters of the ranks are back in step)
    torch.cuda.synchronize()
    host_barrier()
    poller = StatusPoller(dev)
    step(4.0)
    step(5.0)
    poller.flush()
    torch.cuda.synchronize()
    ok = ok and abs(float(g[123]) - 7.5) < 1e-6
    y = float((torch.ones(1024, device=dev) * 2).sum())
    ok = ok and y == 2048.0
    finish(ok)
    """, tmp_path, env_extra={"NCCL_NVLS_ENABLE": "0", "RETURNN_B200_ALLREDUCE_MULTIMEM": "0"})
