"""
Engine end to end on CPU through the public entry point: train the 12AX demo, resume from the checkpoint, forward with a
callback; learning-rate control file; updater options (reference: returnn/torch/engine.py, learning_rate_control.py, torch/updater.py).
"""

import os
import subprocess
import sys
import numpy
import pytest
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, cwd):
    env = dict(os.environ, PYTHONPATH=_ROOT, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, os.path.join(_ROOT, "rnn.py")] + args, cwd=cwd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:] + "\n" + p.stderr[-3000:]
    return p.stdout + p.stderr


def test_train_resume_and_lr_file(tmp_path):
    cfg = os.path.join(_ROOT, "demos", "demo-rf.config")
    model = str(tmp_path / "model")
    lr_file = str(tmp_path / "lr.txt")
    common = [cfg, "++model", model, "++learning_rate_file", lr_file, "++device", "cpu", "++log_verbosity", "4",
              "++train", "{'class': 'Task12AXDataset', 'num_seqs': 200}", "++dev", "{'class': 'Task12AXDataset', 'num_seqs': 40, 'fixed_random_seed': 1}"]
    out1 = _run(common + ["++num_epochs", "2"], str(tmp_path))
    assert os.path.exists(model + ".002.pt") and os.path.exists(model + ".002.opt.pt")
    txt = open(lr_file).read()
    assert "EpochData(learningRate=" in txt and "train_loss_ce" in txt and "dev_loss_ce" in txt
    ck = torch.load(model + ".002.pt", map_location="cpu")
    assert ck["epoch"] == 2 and "model" in ck and any(k.startswith("layers.0") for k in ck["model"])
    step_after_2 = ck["step"]
    out2 = _run(common + ["++num_epochs", "3"], str(tmp_path))
    assert "epoch 3" in out2.lower() or "Epoch 3" in out2
    assert os.path.exists(model + ".003.pt")
    ck3 = torch.load(model + ".003.pt", map_location="cpu")
    assert ck3["epoch"] == 3 and ck3["step"] > step_after_2
    # the score history of epochs 1 and 2 survives the restart
    from returnn_b200.learning_rate_control import load_learning_rate_control_from_config
    from returnn_b200.config import Config

    lrc = load_learning_rate_control_from_config(Config({"learning_rate_file": lr_file, "learning_rate": 0.01}))
    assert set(lrc.epoch_data.keys()) >= {1, 2, 3}


def test_newbob_decays_on_plateau(tmp_path):
    from returnn_b200.learning_rate_control import load_learning_rate_control_from_config
    from returnn_b200.config import Config

    c = Config({"learning_rate": 1.0, "learning_rate_control": "newbob_abs", "newbob_learning_rate_decay": 0.5, "newbob_error_threshold": -0.1,
                "learning_rate_control_relative_error_relative_lr": False})
    lrc = load_learning_rate_control_from_config(c)
    assert lrc.get_learning_rate_for_epoch(1) == 1.0
    lrc.set_epoch_error(1, {"dev_loss": 2.0})
    assert lrc.get_learning_rate_for_epoch(2) == 1.0
    lrc.set_epoch_error(2, {"dev_loss": 1.0})  # improved by 1.0 > threshold: keep
    assert lrc.get_learning_rate_for_epoch(3) == 1.0
    lrc.set_epoch_error(3, {"dev_loss": 0.99})  # improved by less than the threshold: decay
    assert lrc.get_learning_rate_for_epoch(4) == 0.5


def test_updater_param_groups_and_dynamic_lr():
    from returnn_b200.config import Config
    from returnn_b200.torch.updater import Updater

    net = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.LayerNorm(3))
    seen = {}

    def dyn_lr(*, global_train_step, epoch, learning_rate, **_kw):
        seen["step"] = global_train_step
        return learning_rate * 0.5

    cfg = Config({"optimizer": {"class": "adamw", "weight_decay": 0.1, "epsilon": 1e-8}, "dynamic_learning_rate": dyn_lr,
                  "gradient_clip_global_norm": 1.0})
    up = Updater(config=cfg, network=net, device=torch.device("cpu"), initial_learning_rate=0.2)
    up.create_optimizer()
    opt = up.get_optimizer()
    # biases and norm parameters carry no weight decay
    decays = sorted(set(g["weight_decay"] for g in opt.param_groups))
    assert decays == [0.0, 0.1]
    up.set_current_train_step(global_train_step=7, epoch=1, epoch_continuous=0.5)
    assert seen["step"] == 7 and abs(opt.param_groups[0]["lr"] - 0.1) < 1e-9
    before = net[0].weight.detach().clone()
    loss = (net(torch.randn(5, 4)) ** 2).sum() * 100
    opt.zero_grad()
    loss.backward()
    up.step()
    assert not torch.equal(before, net[0].weight)
    assert float(up.get_last_grad_norm()) > 1.0  # the norm before clipping is what gets reported


def test_fused_arena_adamw_matches_torch_adamw_on_cpu():
    from returnn_b200.torch.optim.fused_adamw import FusedArenaAdamW

    torch.manual_seed(0)
    a = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 2))
    b = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 2))
    b.load_state_dict(a.state_dict())
    oa = FusedArenaAdamW(a, lr=1e-2, weight_decay=0.05)
    ob = torch.optim.AdamW(b.parameters(), lr=1e-2, weight_decay=0.05)
    for i in range(5):
        x = torch.randn(7, 6)
        for net, opt in ((a, oa), (b, ob)):
            opt.zero_grad()
            net(x).square().sum().backward()
            opt.step()
    for pa, pb in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(pa, pb, atol=1e-6, rtol=1e-5)
    sd = oa.state_dict()
    assert set(sd["state"][0].keys()) >= {"exp_avg", "exp_avg_sq", "step"}


def test_run_train_step_deferred_losses_match_immediate():
    """``read_losses="deferred"`` hands out the loss of the step before; ``flush_losses`` the last one; same values as reading at once"""
    _deferred_losses_case("cpu")


@pytest.mark.gpu
def test_run_train_step_staged_batches_and_deferred_losses_gpu():
    """the same with the batch copied on the copy stream from pinned memory and the loss read through the pinned ring"""
    _deferred_losses_case("cuda")


def _deferred_losses_case(device):
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Tensor, Dim, batch_dim
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.torch.engine import Engine
    from returnn_b200.datasets.generating import StaticDataset
    from returnn_b200.utils.basic import BehaviorVersion

    time_dim = Dim(None, name="time")
    in_dim, out_dim = Dim(5, name="in"), Dim(3, name="out")

    class Model(rf.Module):
        def __init__(self):
            super().__init__()
            self.lin = rf.Linear(in_dim, out_dim)

    def get_model(**_kw):
        return Model()

    def train_step(*, model, extern_data, **_kw):
        x, y = extern_data["data"], extern_data["classes"]
        logits = model.lin(x)
        loss = rf.cross_entropy(estimated=logits, estimated_type="logits", target=y, axis=out_dim)
        loss.mark_as_loss("ce")

    rng = numpy.random.RandomState(1)
    seqs = [{"data": rng.randn(7, 5).astype("float32"), "classes": rng.randint(0, 3, (7,)).astype("int32")} for _ in range(4)]

    def make_engine():
        cfg = Config({"task": "train", "backend": "torch", "behavior_version": 24, "device": device, "get_model": get_model, "train_step": train_step,
                      "extern_data": {"data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"},
                                      "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32"}},
                      "batch_size": 100, "learning_rate": 0.1, "optimizer": {"class": "sgd"}, "num_epochs": 1, "log_verbosity": 1, "random_seed": 3})
        set_global_config(cfg)
        BehaviorVersion._reset(24)
        data = StaticDataset(data=seqs, output_dim={"data": (5, 2), "classes": (3, 1)})
        data.initialize()
        eng = Engine(cfg)
        eng.init_train_from_config(cfg, data, None, None)
        eng.epoch = 1
        eng._pt_model.train()
        return eng

    def batch(i):
        s = seqs[i]
        res = {"data": torch.from_numpy(s["data"])[None], "classes": torch.from_numpy(s["classes"])[None],
               "data:seq_len": torch.tensor([7], dtype=torch.int32), "classes:seq_len": torch.tensor([7], dtype=torch.int32)}
        if device == "cuda":
            res = {k: (v.pin_memory() if not k.endswith(":seq_len") else v) for k, v in res.items()}
        return res

    eng = make_engine()
    immediate = [eng.run_train_step(batch(i), read_losses=True)["ce"] for i in range(4)]
    eng = make_engine()
    got = []
    for i in range(4):
        res = eng.run_train_step(eng.stage_batch(batch(i)), read_losses="deferred")
        assert (res == {}) == (i == 0)
        if res:
            got.append(res["ce"])
    got.append(eng.flush_losses()["ce"])
    assert eng.flush_losses() == {}
    numpy.testing.assert_allclose(got, immediate, rtol=1e-6 if device == "cpu" else 1e-3)
    assert immediate[-1] < immediate[0] or len(set(immediate)) > 1


def test_prefetch_thread_gives_the_same_training(tmp_path):
    """the background prefetch of batches (default on CUDA) does not change what is trained: same final scores as without it"""
    cfg = os.path.join(_ROOT, "demos", "demo-rf.config")
    scores = []
    for flag in ("False", "True"):
        lr_file = str(tmp_path / ("lr_%s.txt" % flag))
        _run([cfg, "++model", str(tmp_path / ("model_%s" % flag)), "++learning_rate_file", lr_file, "++device", "cpu", "++log_verbosity", "3",
              "++num_epochs", "1", "++torch_dataloader_prefetch_thread", flag, "++train", "{'class': 'Task12AXDataset', 'num_seqs': 120}",
              "++dev", "{'class': 'Task12AXDataset', 'num_seqs': 30, 'fixed_random_seed': 1}"], str(tmp_path))
        from returnn_b200.learning_rate_control import load_learning_rate_control_from_config
        from returnn_b200.config import Config

        lrc = load_learning_rate_control_from_config(Config({"learning_rate_file": lr_file, "learning_rate": 0.01}))
        scores.append(dict(lrc.epoch_data[1].error))
    assert scores[0].keys() == scores[1].keys() and scores[0]
    for k in scores[0]:
        assert abs(scores[0][k] - scores[1][k]) < 1e-6, (k, scores)
