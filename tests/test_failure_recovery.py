"""
Failure detection and recovery, with failures made on the host: a training process that crashes in the middle of an epoch is
restarted by the train process manager and resumes from the last checkpoint; an exception inside a dataset worker process
reaches the main process.
"""

import os
import subprocess
import sys

import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CONFIG = r'''#!rnn.py
import os
from returnn_b200.tensor import Dim, batch_dim
import returnn_b200.frontend as rf

backend = "torch"
task = "train"
device = "cpu"
use_train_proc_manager = True
train = {"class": "Task12AXDataset", "num_seqs": 40}
dev = {"class": "Task12AXDataset", "num_seqs": 10, "fixed_random_seed": 1}
time_dim, in_dim, out_dim = Dim(None, name="time"), Dim(9, name="in"), Dim(2, name="out")
extern_data = {"data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"},
               "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32"}}
batch_size = 2000
optimizer = {"class": "adam"}
learning_rate = 0.01
num_epochs = 3
log_verbosity = 3
model = os.environ["TEST_MODEL_PREFIX"]
_marker = os.environ["TEST_MODEL_PREFIX"] + ".crashed-once"


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        self.lin = rf.Linear(in_dim, out_dim)

    def __call__(self, x):
        return self.lin(x)


def get_model(**_kwargs):
    return Model()


def train_step(*, model, extern_data, **_kwargs):
    ctx = rf.get_run_ctx()
    if ctx.epoch == 2 and not os.path.exists(_marker):
        open(_marker, "w").close()
        os._exit(17)  # the process dies in the middle of epoch 2 (no cleanup, like a kill)
    logits = model(extern_data["data"])
    rf.cross_entropy(estimated=logits, estimated_type="logits", target=extern_data["classes"], axis=out_dim).mark_as_loss("ce")
'''


def test_train_proc_manager_restarts_after_crash(tmp_path):
    cfg = tmp_path / "crash.config"
    cfg.write_text(_CONFIG)
    env = dict(os.environ, TEST_MODEL_PREFIX=str(tmp_path / "net"))
    proc = subprocess.run([sys.executable, os.path.join(_ROOT, "rnn.py"), str(cfg)], cwd=_ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          timeout=600)
    out = proc.stdout.decode("utf8", "replace")
    assert proc.returncode == 0, out[-3000:]
    assert (tmp_path / "net.crashed-once").exists(), "the injected crash did not happen"
    assert "return code 17" in out and "Restarting" in out, out[-3000:]
    for ep in (1, 2, 3):
        assert (tmp_path / ("net.%03d.pt" % ep)).exists(), out[-2000:]
    # the second run resumed at epoch 2 instead of starting over
    assert "Most recent trained model epoch: 1" in out and out.count("start epoch 1 ") <= 1


def _raise_in_worker(seq, **_kwargs):
    if seq.seq_idx == 3:
        raise ValueError("injected failure in the dataset worker")
    return seq


def test_exception_in_dataset_worker_reaches_the_main_process():
    from returnn_b200.datasets.basic import init_dataset

    ds = init_dataset({"class": "MultiProcDataset", "num_workers": 2, "buffer_size": 2,
                       "dataset": {"class": "PostprocessingDataset", "dataset": {"class": "Task12AXDataset", "num_seqs": 12},
                                   "map_seq": _raise_in_worker}})
    try:
        ds.init_seq_order(epoch=1)
        with pytest.raises(Exception) as exc_info:
            i = 0
            while ds.is_less_than_num_seqs(i):
                ds.load_seqs(i, i + 1)
                i += 1
        assert "injected failure" in str(exc_info.value) or "worker" in str(exc_info.value).lower()
    finally:
        ds.finish_epoch(free_resources=True) if hasattr(ds, "finish_epoch") else None
