"""
Failure detection with real GPUs, without a GPU fault: two NCCL ranks (one per GPU) as child processes; rank 1 leaves BETWEEN
two steps, after a device synchronisation (nothing of it is in flight); rank 0 learns of it on the host, from the heartbeat
store, before its next launch, never enters the collective, and its CUDA context stays usable. NVLS is off and the gradient
exchange is plain NCCL (no multicast mappings that a leaving rank could orphan).
"""

import os
import socket
import subprocess
import sys
import textwrap
import pytest
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


_WORKER = """
import os, sys, time
sys.path.insert(0, %r)
import torch, torch.distributed as dist
from returnn_b200.config import Config, set_global_config
from returnn_b200.torch import distributed as rdist
from returnn_b200.parallel.peer_watch import PeerFailure

rank = int(os.environ["RANK"])
torch.cuda.set_device(rank)
cfg = Config({"torch_distributed": {"reduce_type": "grad", "fused": False, "timeout_sec": 60, "peer_watch": {"interval_sec": 0.1, "max_age_sec": 3.0}},
              "log_verbosity": 3})
set_global_config(cfg)
ctx = rdist.get_ctx(cfg)
x = torch.full((1 << 20,), float(rank + 1), device="cuda")
for step in range(3):
    ctx.check_peers(step)
    dist.all_reduce(x)
    torch.cuda.synchronize()
print("rank %%i: 3 steps done, x[0] = %%g" %% (rank, float(x[0])))
if rank == 1:
    ctx.leave_job("test: rank 1 leaves between steps")   # synchronises the device first
    print("rank 1 left")
    sys.stdout.flush()
    os._exit(0)
t0 = time.time()
try:
    for step in range(3, 400):
        ctx.check_peers(step)       # the engine's call before every step: no launch happens after a failure
        time.sleep(0.05)
    print("NOT DETECTED")
except PeerFailure as exc:
    print("DETECTED_ON_HOST ranks=%%s after %%.1f s" %% (exc.ranks, time.time() - t0))
    y = (torch.ones(1024, device="cuda") * 2).sum()
    torch.cuda.synchronize()
    print("CONTEXT_USABLE %%g" %% float(y))
sys.stdout.flush()
os._exit(0)
"""


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_rank_leaving_between_steps_is_detected_on_the_host(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(_WORKER % _ROOT))
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2", LOCAL_WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RETURNN_B200_SMALL_ALLREDUCE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()  # the exact child this test started
            out, _ = p.communicate()
            out += "\n<killed by the test>"
        outs.append((p.returncode, out))
    assert outs[1][0] == 0 and "rank 1 left" in outs[1][1], outs[1][1][-2000:]
    out0 = outs[0][1]
    assert outs[0][0] == 0, out0[-2000:]
    assert "x[0] = " in out0 and "DETECTED_ON_HOST ranks=[1]" in out0 and "CONTEXT_USABLE 2048" in out0, out0[-2000:]
