"""the demo configs train for one epoch on the CPU through the command line entry point (model families end to end)"""

import os
import subprocess
import sys

import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(config, tmp_path, *extra):
    cmd = [sys.executable, os.path.join(_ROOT, "rnn.py"), os.path.join(_ROOT, "demos", config), "++num_epochs", "1", "++device", "cpu",
           "++log_verbosity", "3", "++model", str(tmp_path / "model")] + list(extra)
    proc = subprocess.run(cmd, cwd=_ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=600)
    out = proc.stdout.decode("utf8", "replace")
    assert proc.returncode == 0, out[-3000:]
    assert "Finished training at epoch 1" in out, out[-3000:]
    return out


@pytest.mark.parametrize("config", ["demo-lstm.12ax.config", "demo-blstm-ctc.config", "demo-conformer-ctc.config", "demo-enc-dec-copy.config",
                                    "demo-pretrain.config", "demo-rf.config", "demo-torch.config"])
def test_demo_trains_one_epoch(config, tmp_path):
    out = _run(config, tmp_path)
    assert (tmp_path / "model.001.pt").exists(), out[-2000:]


def test_forward_task_and_priors(tmp_path):
    """train one epoch, then task=forward with a callback and task=compute_priors from the checkpoint"""
    _run("demo-lstm.12ax.config", tmp_path, "++train", '{"class": "Task12AXDataset", "num_seqs": 60}')
    prior_file = tmp_path / "priors.txt"
    cmd = [sys.executable, os.path.join(_ROOT, "rnn.py"), os.path.join(_ROOT, "demos", "demo-lstm.12ax.config"), "++task", "compute_priors", "++device", "cpu",
           "++load", str(tmp_path / "model.001"), "++train", '{"class": "Task12AXDataset", "num_seqs": 20}', "++output_file", str(prior_file),
           "++log_verbosity", "3", "++forward_callback", "None"]
    proc = subprocess.run(cmd, cwd=_ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=600)
    out = proc.stdout.decode("utf8", "replace")
    assert proc.returncode == 0, out[-3000:]
    vals = [float(x) for x in prior_file.read_text().split()]
    assert len(vals) == 2 and abs(sum(2.718281828 ** v for v in vals) - 1.0) < 1e-3


@pytest.mark.parametrize("script", ["demo-sprint-interface.py", "demo-push-to-webserver.py"])
def test_demo_scripts_run(script):
    """the stand-alone demo scripts (producer-fed dataset through a child process; HTTP client against an in-process server)"""
    import os
    import subprocess
    import sys

    demos = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "demos")
    res = subprocess.run([sys.executable, script], cwd=demos, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    if "sprint" in script:
        assert "epoch 2 seq 4" in res.stdout and "data (" in res.stdout
    else:
        assert "output 'output': (7, 2)" in res.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("config", ["demo-lstm.12ax.config", "demo-blstm-ctc.config", "demo-conformer-ctc.config", "demo-enc-dec-copy.config", "demo-rf.config",
                                    "demo-torch.config"])
def test_demo_trains_one_epoch_on_the_gpu(config, tmp_path):
    """the same configs on the GPU: the generic RF path on the own kernels (LSTM with 9 inputs and 100 units, odd widths, small vocabularies)"""
    cmd = [sys.executable, os.path.join(_ROOT, "rnn.py"), os.path.join(_ROOT, "demos", config), "++num_epochs", "1", "++device", "cuda", "++log_verbosity", "3",
           "++model", str(tmp_path / "model")]
    proc = subprocess.run(cmd, cwd=_ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=900)
    out = proc.stdout.decode("utf8", "replace")
    assert proc.returncode == 0 and "Finished training at epoch 1" in out, out[-3000:]
    assert (tmp_path / "model.001.pt").exists()
