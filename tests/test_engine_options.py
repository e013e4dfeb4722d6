"""
Engine options, each on a tiny frame-classification task on the CPU, in process: gradient accumulation, clipping, learning-rate lists
and control, checkpoint interval / cleanup / import / preload, sequence length filters, chunking, evaluation datasets, non-finite
losses, forward with a callback (reference: returnn/torch/engine.py, tests/test_torch_engine.py).
"""

import os
import numpy
import pytest
import torch

import returnn_b200.frontend as rf
from returnn_b200.tensor import Tensor, Dim, batch_dim
from returnn_b200.config import Config, set_global_config
from returnn_b200.utils.basic import BehaviorVersion
from returnn_b200.torch.engine import Engine
from returnn_b200.datasets.generating import StaticDataset

time_dim = Dim(None, name="time")
in_dim = Dim(5, name="in")
out_dim = Dim(3, name="out")
EXTERN = {"data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"}, "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32"}}


class Model(rf.Module):
    def __init__(self):
        super().__init__()
        self.hidden = rf.Linear(in_dim, Dim(8, name="hid"))
        self.out = rf.Linear(self.hidden.out_dim, out_dim)

    def __call__(self, x):
        return self.out(rf.tanh(self.hidden(x)))


def get_model(**_kw):
    return Model()


def train_step(*, model, extern_data, **_kw):
    logits = model(extern_data["data"])
    ce = rf.cross_entropy(estimated=logits, estimated_type="logits", target=extern_data["classes"], axis=out_dim)
    ce.mark_as_loss("ce")
    err = rf.reduce_argmax(logits, axis=out_dim) != extern_data["classes"]
    err.mark_as_loss("fer", as_error=True)


def forward_step(*, model, extern_data, **_kw):
    rf.softmax(model(extern_data["data"]), axis=out_dim).mark_as_default_output(shape=[batch_dim, time_dim, out_dim])


def _seqs(n, seed=1, min_len=4, max_len=9):
    rng = numpy.random.RandomState(seed)
    w = numpy.random.RandomState(0).randn(5, 3)
    out = []
    for _ in range(n):
        t = int(rng.randint(min_len, max_len + 1))
        x = rng.randn(t, 5).astype("float32")
        out.append({"data": x, "classes": numpy.argmax(x @ w, axis=1).astype("int32")})
    return out


def _dataset(seqs, **kw):
    d = StaticDataset(data=seqs, output_dim={"data": (5, 2), "classes": (3, 1)}, **kw)
    d.initialize()
    return d


def _engine(tmp_path, *, train=None, dev=None, **opts):
    cfg = Config(dict({"task": "train", "backend": "torch", "behavior_version": 24, "device": "cpu", "get_model": get_model, "train_step": train_step,
                       "forward_step": forward_step, "extern_data": EXTERN, "batch_size": 60, "max_seqs": 8, "learning_rate": 0.05,
                       "optimizer": {"class": "adam"}, "num_epochs": 2, "log_verbosity": 2, "random_seed": 3, "model": str(tmp_path / "model"),
                       "learning_rate_file": str(tmp_path / "lr.txt")}, **opts))
    set_global_config(cfg)
    BehaviorVersion._reset(24)
    eng = Engine(cfg)
    eng.init_train_from_config(cfg, train if train is not None else _dataset(_seqs(24)), dev, None)
    return eng, cfg


def _params(eng):
    return {k: v.detach().clone() for k, v in eng._pt_model.state_dict().items()}


def test_training_reduces_the_loss_and_writes_checkpoints(tmp_path):
    eng, _ = _engine(tmp_path, dev=_dataset(_seqs(8, seed=5)), num_epochs=4)
    eng.train()
    data = eng.learning_rate_control.epoch_data
    assert data[4].error["train_loss_ce"] < data[1].error["train_loss_ce"] and "dev_loss_ce" in data[4].error and "dev_loss_fer" in data[4].error
    for ep in (1, 2, 3, 4):
        assert os.path.exists(str(tmp_path / ("model.%03i.pt" % ep)))


@pytest.mark.parametrize("interval", [2, 3])
def test_save_interval(tmp_path, interval):
    eng, _ = _engine(tmp_path, num_epochs=4, save_interval=interval)
    eng.train()
    have = sorted(int(f.split(".")[1]) for f in os.listdir(tmp_path) if f.startswith("model.") and f.endswith(".pt") and ".opt." not in f)
    assert have == sorted({e for e in range(1, 5) if e % interval == 0} | {4})  # the last epoch is always saved


def test_cleanup_old_models_keeps_last_and_best(tmp_path):
    eng, _ = _engine(tmp_path, dev=_dataset(_seqs(8, seed=5)), num_epochs=6, cleanup_old_models={"keep_last_n": 2, "keep_best_n": 1, "keep": [1]})
    eng.train()
    have = sorted(int(f.split(".")[1]) for f in os.listdir(tmp_path) if f.startswith("model.") and f.endswith(".pt") and ".opt." not in f)
    assert 1 in have and 5 in have and 6 in have and len(have) <= 4


def test_accum_grad_multiple_step_equals_one_large_batch(tmp_path):
    """two sequences per step with an update every second step == four sequences per step, for SGD and a summed loss: the gradients of the
    accumulated steps add up (they are not averaged)"""
    seqs = _seqs(8, min_len=6, max_len=6)

    def summed_train_step(*, model, extern_data, **_kw):
        logits = model(extern_data["data"])
        rf.cross_entropy(estimated=logits, estimated_type="logits", target=extern_data["classes"], axis=out_dim).mark_as_loss("ce")

    res = []
    for max_seqs, accum in ((4, 1), (2, 2)):
        eng, _ = _engine(tmp_path / ("a%i" % accum), train=_dataset(seqs), num_epochs=1, max_seqs=max_seqs, accum_grad_multiple_step=accum,
                         optimizer={"class": "sgd"}, learning_rate=0.01, train_step=summed_train_step)
        eng.train()
        res.append(_params(eng))
    for k in res[0]:
        torch.testing.assert_close(res[0][k], res[1][k], atol=1e-6, rtol=1e-5)


def test_gradient_clip_global_norm_bounds_the_update(tmp_path):
    moved = []
    for clip in (0.0, 1e-3):
        eng, _ = _engine(tmp_path / ("c%s" % clip), num_epochs=1, optimizer={"class": "sgd"}, learning_rate=1.0, gradient_clip_global_norm=clip, max_seqs=100,
                         batch_size=10000)
        before = _params(eng)
        eng.train()
        after = _params(eng)
        moved.append(float(torch.sqrt(sum(((after[k] - before[k]) ** 2).sum() for k in before))))
    assert moved[1] <= 1e-3 * 1.0001 and moved[0] > 10 * moved[1]  # one step of lr 1: the update norm is the clipped gradient norm


def test_learning_rates_list_then_control(tmp_path):
    eng, _ = _engine(tmp_path, num_epochs=4, learning_rates=[0.001, 0.002, 0.003], learning_rate=0.01)
    eng.train()
    lrs = [eng.learning_rate_control.epoch_data[e].learning_rate for e in (1, 2, 3, 4)]
    assert lrs[:3] == [0.001, 0.002, 0.003] and lrs[3] == pytest.approx(0.003)  # constant control continues with the last value


def test_newbob_control_through_the_engine(tmp_path):
    """a relative threshold that no run can meet: the rate halves after every epoch with a dev score"""
    eng, _ = _engine(tmp_path, dev=_dataset(_seqs(8, seed=5)), num_epochs=3, learning_rate_control="newbob_rel", newbob_relative_error_threshold=-10.0,
                     newbob_learning_rate_decay=0.5, learning_rate_control_min_num_epochs_per_new_lr=0, learning_rate=0.04,
                     learning_rate_control_relative_error_relative_lr=False)
    eng.train()
    lrs = [eng.learning_rate_control.epoch_data[e].learning_rate for e in (1, 2, 3)]
    assert lrs[0] == 0.04 and lrs[2] < lrs[0] and lrs[2] in (0.02, 0.01)


def test_resume_continues_epoch_and_step(tmp_path):
    eng, _ = _engine(tmp_path, num_epochs=2)
    eng.train()
    step2 = eng.global_train_step
    eng2, _ = _engine(tmp_path, num_epochs=3)
    assert eng2.start_epoch == 3 if hasattr(eng2, "start_epoch") else True
    eng2.train()
    assert eng2.global_train_step > step2 and os.path.exists(str(tmp_path / "model.003.pt"))
    ck = torch.load(str(tmp_path / "model.003.pt"), map_location="cpu")
    assert ck["epoch"] == 3 and ck["step"] == eng2.global_train_step


def test_import_model_train_epoch1_and_preload_from_files(tmp_path):
    src, _ = _engine(tmp_path / "src", num_epochs=1)
    src.train()
    src_params = torch.load(str(tmp_path / "src" / "model.001.pt"), map_location="cpu")["model"]
    eng, _ = _engine(tmp_path / "imp", num_epochs=1, import_model_train_epoch1=str(tmp_path / "src" / "model.001"), learning_rate=0.0,
                     optimizer={"class": "sgd"})
    for k, v in _params(eng).items():
        torch.testing.assert_close(v, src_params[k])
    # a checkpoint of one sub-module (keys without the sub-module's name) goes under a prefix; the rest keeps its own initialisation
    torch.save({"model": {"weight": src_params["hidden.weight"], "bias": src_params["hidden.bias"]}, "epoch": 1, "step": 0}, str(tmp_path / "hidden_only.pt"))
    eng2, _ = _engine(tmp_path / "pre", num_epochs=1, random_seed=99,
                      preload_from_files={"first": {"filename": str(tmp_path / "hidden_only.pt"), "prefix": "hidden.", "init_for_train": True}})
    p2 = _params(eng2)
    torch.testing.assert_close(p2["hidden.weight"], src_params["hidden.weight"])
    assert not torch.equal(p2["out.weight"], src_params["out.weight"])


@pytest.mark.parametrize("opts,expect", [({"max_seq_length": {"data": 6}}, lambda n: n <= 6), ({"min_seq_length": {"data": 7}}, lambda n: n >= 7)])
def test_sequence_length_filters(tmp_path, opts, expect):
    seqs = _seqs(30)
    seen = []

    def spy_train_step(*, model, extern_data, **kw):
        seen.extend(extern_data["data"].dims[1].dyn_size_ext.raw_tensor.tolist())
        train_step(model=model, extern_data=extern_data)

    eng, _ = _engine(tmp_path, train=_dataset(seqs), num_epochs=1, train_step=spy_train_step, **opts)
    eng.train()
    want = [s["data"].shape[0] for s in seqs if expect(s["data"].shape[0])]
    assert sorted(seen) == sorted(want) and 0 < len(seen) < len(seqs)


def test_chunking_cuts_sequences(tmp_path):
    seqs = _seqs(6, min_len=20, max_len=20)
    seen = []

    def spy_train_step(*, model, extern_data, **kw):
        seen.extend(extern_data["data"].dims[1].dyn_size_ext.raw_tensor.tolist())
        train_step(model=model, extern_data=extern_data)

    eng, _ = _engine(tmp_path, train=_dataset(seqs), num_epochs=1, train_step=spy_train_step, chunking="8:8")
    eng.train()
    assert sorted(seen) == sorted([8, 8, 4] * 6)


def test_eval_datasets_are_scored_every_epoch(tmp_path):
    eng, cfg = _engine(tmp_path, num_epochs=2, eval_datasets={"devtrain": {"class": "StaticDataset", "data": _seqs(5, seed=7), "output_dim": {"data": (5, 2), "classes": (3, 1)}}})
    eng.train()
    err = eng.learning_rate_control.epoch_data[2].error
    assert "devtrain_loss_ce" in err and "devtrain_loss_fer" in err and 0.0 <= err["devtrain_loss_fer"] <= 1.0


def test_nonfinite_loss_stops_training(tmp_path):
    def bad_train_step(*, model, extern_data, **kw):
        logits = model(extern_data["data"])
        ce = rf.cross_entropy(estimated=logits, estimated_type="logits", target=extern_data["classes"], axis=out_dim)
        (ce * float("nan")).mark_as_loss("ce")

    eng, _ = _engine(tmp_path, num_epochs=1, train_step=bad_train_step, stop_on_nonfinite_train_score=True)
    with pytest.raises(Exception, match="(?i)nan|inf|finite"):
        eng.train()


def test_forward_with_callback_covers_every_sequence(tmp_path):
    from returnn_b200.forward_iface import ForwardCallbackIface

    eng, _ = _engine(tmp_path, num_epochs=1)
    eng.train()
    seqs = _seqs(7, seed=11)
    got = {}

    class Collect(ForwardCallbackIface):
        def init(self, *, model):
            got["init"] = True

        def process_seq(self, *, seq_tag, outputs):
            got[seq_tag] = outputs["output"].raw_tensor

        def finish(self):
            got["finish"] = True

    eng.forward_with_callback(dataset=_dataset(seqs), callback=Collect())
    assert got.pop("init") and got.pop("finish") and len(got) == 7
    for i, s in enumerate(seqs):
        p = got["seq-%i" % i]
        assert p.shape == (s["data"].shape[0], 3)
        numpy.testing.assert_allclose(numpy.asarray(p).sum(-1), 1.0, atol=1e-5)


def test_dynamic_learning_rate_sees_every_step(tmp_path):
    seen = []

    def dyn(*, global_train_step, epoch, learning_rate, **kw):
        seen.append((global_train_step, epoch))
        return learning_rate * 0.1

    eng, _ = _engine(tmp_path, num_epochs=2, dynamic_learning_rate=dyn)
    eng.train()
    steps = [s for s, _ in seen]
    assert steps == sorted(steps) and steps[-1] >= eng.global_train_step - 1 and {e for _, e in seen} == {1, 2}
