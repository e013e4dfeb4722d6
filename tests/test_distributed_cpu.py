"""
Data-parallel logic on CPU with gloo, 2 ranks as child processes: the three reduce types give the documented results,
the bucketed reducer handles gradients written outside autograd, and a rank that fails is detected by the others
through a short process-group timeout (the failure is made on the host).
"""

import os
import socket
import sys
import textwrap
import subprocess
import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(body: str, tmp_path, world=2, timeout=300, expect_ok=True):
    script = tmp_path / "worker.py"
    script.write_text("import os, sys\nsys.path.insert(0, %r)\n" % _ROOT + textwrap.dedent(body))
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<killed by the test after %i s>" % timeout
        outs.append((p.returncode, out))
    if expect_ok:
        for rc, out in outs:
            assert rc == 0, out[-3000:]
    return outs


_COMMON = """
import torch, torch.distributed as dist
from returnn_b200.config import Config, set_global_config
from returnn_b200.torch import distributed as rdist

def make_ctx(opts):
    cfg = Config({"torch_distributed": opts, "log_verbosity": 3})
    set_global_config(cfg)
    return rdist.get_ctx(cfg)

def model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
"""


@pytest.mark.parametrize("reduce_type", ["grad", "grad_explicit"])
def test_grad_reduce_types_average_gradients(tmp_path, reduce_type):
    outs = _launch(_COMMON + """
ctx = make_ctx({"reduce_type": %r})
rank, world = ctx.rank(), ctx.size()
net = model()
ctx.setup_grad_reduction(net)
torch.manual_seed(100 + rank)
x = torch.randn(5, 8)
ctx.prepare_backward(sync=True)
net(x).square().sum().backward()
ctx.maybe_reduce_grads(net)
mine = torch.cat([p.grad.reshape(-1) for p in net.parameters()])
# reference: average of the two ranks' local gradients, recomputed here without any reduction
ref = 0
for r in range(world):
    n2 = model()
    torch.manual_seed(100 + r)
    n2(torch.randn(5, 8)).square().sum().backward()
    ref = ref + torch.cat([p.grad.reshape(-1) for p in n2.parameters()]) / world
assert torch.allclose(mine, ref, atol=1e-6), (mine - ref).abs().max()
print("OK", rank)
dist.destroy_process_group()
""" % reduce_type, tmp_path)
    assert all("OK" in o for _, o in outs)


@pytest.mark.parametrize("zero_mode", ["updater", "set_to_none"])
def test_grad_reduction_with_torch_sgd_over_several_steps(tmp_path, zero_mode):
    """
    A plain torch optimizer (no arena optimizer): after every step the gradients each rank applies must be the average over the
    ranks, also when the gradients were set to None before backward, so that autograd allocates tensors outside the arena.
    """
    outs = _launch(_COMMON + """
from returnn_b200.torch.updater import Updater
zero_mode = %r
ctx = make_ctx({"reduce_type": "grad", "bucket_cap_mb": 0})
rank, world = ctx.rank(), ctx.size()
net = model()
ctx.setup_grad_reduction(net)
cfg = Config({"optimizer": {"class": "sgd"}, "learning_rate": 0.1})
upd = Updater(config=cfg, network=net, device=torch.device("cpu"), initial_learning_rate=0.1)
upd.set_arena(ctx.arena)
upd.create_optimizer()
assert not getattr(upd.get_optimizer(), "is_fused_arena", False)
# the same training done by hand: every rank's data on one model, gradient = average over the ranks
ref = model()
for step in range(3):
    if zero_mode == "updater":
        upd.zero_grad()
    else:
        upd.get_optimizer().zero_grad(set_to_none=True)
    torch.manual_seed(1000 * step + rank)
    x = torch.randn(5, 8)
    ctx.prepare_backward(sync=True)
    net(x).square().sum().backward()
    ctx.maybe_reduce_grads(net)
    mine = torch.cat([p.grad.reshape(-1) for p in net.parameters()]).clone()
    upd.step()
    for p in ref.parameters():
        p.grad = None
    for r in range(world):
        torch.manual_seed(1000 * step + r)
        (ref(torch.randn(5, 8)).square().sum() / world).backward()
    want = torch.cat([p.grad.reshape(-1) for p in ref.parameters()])
    assert torch.allclose(mine, want, atol=1e-5), (step, float((mine - want).abs().max()))
    with torch.no_grad():
        for p in ref.parameters():
            p.sub_(0.1 * p.grad)
    for p, q in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-5), (step, float((p - q).abs().max()))
print("OK", rank)
dist.destroy_process_group()
""" % zero_mode, tmp_path)
    assert all("OK" in o for _, o in outs)


def test_param_averaging(tmp_path):
    outs = _launch(_COMMON + """
ctx = make_ctx({"reduce_type": "param", "param_sync_step": 2})
rank, world = ctx.rank(), ctx.size()
net = model()
ctx.setup_grad_reduction(net)
with torch.no_grad():
    for p in net.parameters():
        p.add_(float(rank))
assert not ctx.should_sync_now(epoch_step_idx=0) and ctx.should_sync_now(epoch_step_idx=1)
ctx.step_after_param_update(module=net, epoch_step_idx=1)
ref = model()
for p, q in zip(net.parameters(), ref.parameters()):
    assert torch.allclose(p, q + 0.5, atol=1e-6)
print("OK", rank)
dist.destroy_process_group()
""", tmp_path)
    assert all("OK" in o for _, o in outs)


def test_reducer_with_gradients_written_outside_autograd(tmp_path):
    outs = _launch(_COMMON + """
from returnn_b200.parallel import grad_reducer
ctx = make_ctx({"reduce_type": "grad", "bucket_cap_mb": 0})
rank, world = ctx.rank(), ctx.size()
net = model()
ctx.setup_grad_reduction(net)
arena = ctx.arena
assert arena is not None and len(arena.buckets) >= 2
ctx.prepare_backward(sync=True)
# first layer through autograd, second layer's gradients written by hand into the arena and announced
x = torch.randn(3, 8)
h = net[1](net[0](x)).sum()
h.backward()
w2, b2 = net[2].weight, net[2].bias
w2.grad.fill_(1.0 + rank)
b2.grad.fill_(10.0 * (1 + rank))
grad_reducer.notify_grads_written([w2, b2])
ctx.maybe_reduce_grads(net)
assert torch.allclose(w2.grad, torch.full_like(w2.grad, 1.5)), w2.grad
assert torch.allclose(b2.grad, torch.full_like(b2.grad, 15.0))
print("OK", rank)
dist.destroy_process_group()
""", tmp_path)
    assert all("OK" in o for _, o in outs)


def test_failed_rank_is_detected_by_timeout(tmp_path):
    outs = _launch("""
import datetime, time, torch, torch.distributed as dist
rank = int(os.environ["RANK"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
t = torch.ones(4)
dist.all_reduce(t)
if rank == 1:
    print("rank 1 leaves between steps")
    os._exit(3)
try:
    dist.all_reduce(t)
    print("NO ERROR")
except Exception as exc:
    print("DETECTED", type(exc).__name__)
""", tmp_path, expect_ok=False, timeout=120)
    rc0, out0 = outs[0]
    assert "DETECTED" in out0 and "NO ERROR" not in out0, out0
    assert outs[1][0] == 3


def test_peer_watch_states_with_fake_store_and_clock():
    """alive -> stale -> PeerFailure; a rank that leaves on purpose is reported at once"""
    from returnn_b200.parallel.peer_watch import PeerWatch, PeerFailure

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

        def check(self, keys):
            return all(k in self for k in keys)

    now = [100.0]
    store = Store()
    w0 = PeerWatch(store, rank=0, world=2, max_age_sec=5.0, clock=lambda: now[0], start_thread=False)
    assert w0.failed_ranks() == {1: "no heartbeat entry"}
    w1 = PeerWatch(store, rank=1, world=2, max_age_sec=5.0, clock=lambda: now[0], start_thread=False)
    w0.check(step=1)
    now[0] += 3.0
    w1.beat(step=7)
    now[0] += 4.0
    w0.check(step=2)  # 4 s old: fine
    assert w0.status()[1]["step"] == 7
    now[0] += 2.0
    with pytest.raises(PeerFailure) as exc:
        w0.check(step=3)
    assert exc.value.ranks == [1] and "step 7" in exc.value.reasons[1]
    w1.beat()
    w0.check()
    w1.leave("node drained")
    with pytest.raises(PeerFailure) as exc:
        w0.check()
    assert "node drained" in exc.value.reasons[1]


def test_peer_that_leaves_is_detected_on_the_host_before_the_next_collective(tmp_path):
    """rank 1 leaves between two steps; rank 0 learns of it from the store and never enters the collective (no timeout wait)"""
    outs = _launch(_COMMON + """
import time
rank = int(os.environ["RANK"])
ctx = make_ctx({"reduce_type": "grad", "timeout_sec": 600, "peer_watch": {"interval_sec": 0.1, "max_age_sec": 3.0}})
from returnn_b200.parallel.peer_watch import PeerFailure
t = torch.ones(4)
ctx.check_peers(0)
dist.all_reduce(t)
if rank == 1:
    ctx.leave_job("test: leaving between steps")
    print("rank 1 left")
    os._exit(0)
t0 = time.time()
try:
    for step in range(1, 200):
        ctx.check_peers(step)      # what the engine does before every step
        time.sleep(0.05)
    print("NOT DETECTED")
except PeerFailure as exc:
    print("DETECTED_ON_HOST ranks=%s after %.1f s: %s" % (exc.ranks, time.time() - t0, exc))
os._exit(0)
""", tmp_path, expect_ok=False, timeout=120)
    rc0, out0 = outs[0]
    assert "DETECTED_ON_HOST ranks=[1]" in out0 and "leaving between steps" in out0, out0
    assert outs[1][0] == 0 and "rank 1 left" in outs[1][1]


def test_peer_that_dies_silently_is_detected_by_stale_heartbeat(tmp_path):
    """rank 1 exits without a word (its heartbeat thread dies with it): rank 0 sees the heartbeat age out"""
    outs = _launch(_COMMON + """
import time
rank = int(os.environ["RANK"])
ctx = make_ctx({"reduce_type": "grad", "timeout_sec": 600, "peer_watch": {"interval_sec": 0.1, "max_age_sec": 1.5}})
from returnn_b200.parallel.peer_watch import PeerFailure
t = torch.ones(4)
dist.all_reduce(t)
if rank == 1:
    os._exit(7)
try:
    for step in range(1, 400):
        ctx.check_peers(step)
        time.sleep(0.05)
    print("NOT DETECTED")
except PeerFailure as exc:
    print("DETECTED_ON_HOST", exc)
os._exit(0)
""", tmp_path, expect_ok=False, timeout=120)
    rc0, out0 = outs[0]
    assert "DETECTED_ON_HOST" in out0 and "last heartbeat" in out0, out0
    assert outs[1][0] == 7
