"""
The RASR criterion bridge: ``sprint.error_signals`` (trainer side) against ``sprint.control`` (the module RASR loads), with a stand-in
executable that loads the module from its ``--*.pymod-*`` arguments and calls it the way RASR's PythonControl does. The stand-in's
criterion is a frame-wise cross entropy against an alignment derived from the segment name, so loss and error signal are known.
"""

import os
import stat
import sys
import textwrap
import numpy
import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _targets(name: str, n: int, dim: int):
    seed = sum(ord(c) for c in name)
    return (numpy.arange(n) * 7 + seed) % dim


def _stand_in_exec(tmp_path, mode="control-loop"):
    """
    mode "control-loop": RASR hands its thread to ``run_control_loop`` and answers through its callback.
    mode "segment-order": RASR iterates ``getSegmentList`` and its trainer uses the NnPythonLayer calls per segment.
    """
    path = tmp_path / ("fake-rasr-%s" % mode)
    path.write_text("#!%s\n" % sys.executable + textwrap.dedent('''
        import importlib, sys, time
        import numpy
        args = dict(a[4:].split("=", 1) for a in sys.argv[1:] if a.startswith("--*.") and "=" in a)
        sys.path.insert(0, args["pymod-path"])
        mod = importlib.import_module(args["pymod-name"])
        slow = float(args.get("slow-instance-seconds", "0"))

        def targets(name, n, dim):
            seed = sum(ord(c) for c in name)
            return (numpy.arange(n) * 7 + seed) % dim

        def criterion(name, log_post):
            n, dim = log_post.shape
            if "fail" in name:
                raise ValueError("no path for " + name)
            t = targets(name, n, dim)
            loss = -float(log_post[numpy.arange(n), t].sum())
            err = numpy.exp(log_post)
            err[numpy.arange(n), t] -= 1.0
            time.sleep(slow * n / 100.0)
            return loss, err.astype("float32")

        def callback(action, *a, **kw):
            if action == "version":
                return "<version>fake</version>"
            if action == "get_loss_and_error_signal":
                name, n, post = a
                return criterion(name, post)
            if action == "export_allophone_state_fsa_by_segment_name":
                (name,) = a
                n = 2 + len(name) % 3  # a chain of n states: edge i -> i+1 with emission i
                edges = numpy.array([list(range(n - 1)), list(range(1, n)), list(range(n - 1))], dtype="uint32").reshape(-1)
                return n, n - 1, edges, numpy.full((n - 1,), 0.5, dtype="float32")
            raise NotImplementedError(action)

        MODE = @MODE@
        if MODE == "control-loop":
            ctl = mod.init(name="Sprint.PythonControl", reference=object(), config=args["pymod-config"], sprint_unit="NnTrainer.pythonControl",
                           version_number=5, callback=callback)
            ctl.init_processing(input_dim=3, output_dim=4)
            try:
                ctl.run_control_loop(callback)
            except SystemExit:
                pass
            ctl.exit()
        else:
            assert args["python-segment-order"] == "true"
            layer = None
            for seg in mod.getSegmentList("corpus", [], config=args["python-segment-order-config"]):
                ctl = mod.PythonControl.instance
                if layer is None:
                    layer = mod.SprintNnPythonLayer(config=args["pymod-config"])
                    layer.setInputDimension(0, 3)
                if "skip" in seg:
                    continue  # RASR drops the segment without touching it
                ctl.init_segment(seg)
                n = ctl.seg_len
                layer.setOutputDimension(ctl.posteriors.shape[1])
                post = layer.forward((numpy.zeros((3, n), "float32"),))  # (D, T)
                loss, err = criterion(seg, numpy.ascontiguousarray(post.T))
                ctl.notify_segment_loss(seg, loss)
                (back,) = layer.backpropagate(numpy.ascontiguousarray(err.T))
                assert back.shape == (3, n)
        ''').replace("@MODE@", repr(mode)))
    path.chmod(path.stat().st_mode | stat.S_IXUSR)
    return str(path)


def _batch(rng, lens, dim):
    x = rng.randn(max(lens), len(lens), dim).astype("float32")
    x = x - numpy.log(numpy.exp(x).sum(-1, keepdims=True))
    return x


def _expected(x, lens, tags):
    loss = numpy.zeros(len(lens), "float32")
    err = numpy.zeros_like(x)
    for b, (n, tag) in enumerate(zip(lens, tags)):
        t = _targets(tag, n, x.shape[-1])
        loss[b] = -x[numpy.arange(n), b, t].sum()
        err[:n, b] = numpy.exp(x[:n, b])
        err[numpy.arange(n), b, t] -= 1
    return loss, err


@pytest.mark.parametrize("num_instances", [1, 3])
def test_pool_batch_loss_and_error_signal(tmp_path, num_instances):
    from returnn_b200.sprint.error_signals import SprintInstancePool

    pool = SprintInstancePool({"sprintExecPath": _stand_in_exec(tmp_path), "numInstances": num_instances, "sprintConfigStr": "--*.slow-instance-seconds=0.02",
                               "sprintControlConfig": {"quiet": True}})
    try:
        rng = numpy.random.RandomState(1)
        for step in range(2):  # the children live across batches
            lens = [9, 17, 4, 12, 17, 6, 3][: 7 - step]
            tags = ["corpus/rec/seg-%i-%i" % (step, i) for i in range(len(lens))]
            x = _batch(rng, lens, dim=5)
            loss, err = pool.get_batch_loss_and_error_signal(x, numpy.array(lens, "int32"), tags)
            want_loss, want_err = _expected(x, lens, tags)
            numpy.testing.assert_allclose(loss, want_loss, rtol=1e-5)
            numpy.testing.assert_allclose(err, want_err, atol=1e-6)
        assert len(pool.instances) == num_instances
        # a segment RASR fails on gives an error here, and the child stays usable
        with pytest.raises(RuntimeError, match="no path"):
            pool.get_batch_loss_and_error_signal(x[:, :1], numpy.array(lens[:1], "int32"), ["seg-fail"])
        loss, _ = pool.get_batch_loss_and_error_signal(x[:, :1], numpy.array(lens[:1], "int32"), tags[:1])
        numpy.testing.assert_allclose(loss, want_loss[:1], rtol=1e-5)
        # automata of a batch, merged into one state space
        edges, weights, start_end = pool.get_automata_for_batch(["ab", "abc", "a"])
        n_states = [2 + 2 % 3, 2 + 3 % 3, 2 + 1 % 3]
        assert edges.shape == (4, sum(n - 1 for n in n_states)) and weights.shape == (edges.shape[1],)
        assert start_end.tolist() == [[0, 4, 6], [3, 5, 8]]
        assert edges[3].tolist() == [0, 0, 0, 1, 2, 2] and edges[0].tolist() == [0, 1, 2, 4, 6, 7] and edges[2].tolist() == [0, 1, 2, 0, 0, 1]
    finally:
        pool.close()


def test_sprint_loss_autograd_and_segment_order_mode(tmp_path):
    """through autograd; RASR drives (python segment order + NnPythonLayer), one of the segments is skipped by RASR"""
    import torch
    from returnn_b200.sprint.error_signals import sprint_loss, SprintInstancePool

    opts = {"sprintExecPath": _stand_in_exec(tmp_path, "segment-order"), "numInstances": 2, "sprintControlConfig": {"quiet": True}}
    try:
        rng = numpy.random.RandomState(2)
        lens = [8, 5, 11]
        tags = ["s0", "s1-skip", "s2"]
        logits = torch.tensor(rng.randn(3, 11, 6).astype("float32"), requires_grad=True)
        log_probs = torch.log_softmax(logits, -1)
        loss = sprint_loss(log_probs, torch.tensor(lens), tags, opts)
        want_loss, want_err = _expected(log_probs.detach().numpy().transpose(1, 0, 2), lens, tags)
        want_loss[1] = 0.0  # the skipped segment: no loss, no gradient
        want_err[:, 1] = 0.0
        numpy.testing.assert_allclose(loss.detach().numpy(), want_loss, rtol=1e-5)
        scale = torch.tensor([1.0, 1.0, 0.5])
        (g,) = torch.autograd.grad((loss * scale).sum(), log_probs)
        numpy.testing.assert_allclose(g.numpy(), want_err.transpose(1, 0, 2) * scale.numpy()[:, None, None], atol=1e-6)
    finally:
        SprintInstancePool.get_global_instance(opts).close()


# ---- this framework inside a RASR process (sprint.interface) ----

_INTERFACE_CONFIG = '''
import torch
import returnn_b200.frontend as rf

backend = "torch"
device = "cpu"
extern_data = {"data": {"dim": 5}, "classes": {"dim": 3, "sparse": True, "available_for_inference": False}}
model_outputs = {"output": {"dim": 3}}
batching = "random"
batch_size = 500
max_seqs = 4
optimizer = {"class": "adam"}
learning_rate = 0.05
num_epochs = 3
log_verbosity = 3
model = "@MODEL@"


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = torch.nn.Linear(5, 3)

    def forward(self, x):
        return self.lin(x)


def get_model(**_kwargs):
    return Net()


def train_step(*, model, extern_data, **_kwargs):
    data, targets = extern_data["data"], extern_data["classes"]
    logits = model(data.raw_tensor)
    lens = data.dims[1].dyn_size_ext.raw_tensor
    mask = torch.arange(logits.shape[1])[None, :] < lens[:, None]
    ce = torch.nn.functional.cross_entropy(logits[mask], targets.raw_tensor[mask].long(), reduction="none")
    rf.get_run_ctx().mark_as_loss(name="ce", loss=ce)


def forward_step(*, model, extern_data, **_kwargs):
    data = extern_data["data"]
    out = torch.softmax(model(data.raw_tensor), -1)
    ctx = rf.get_run_ctx()
    ctx.expected_outputs["output"].dims[1].dyn_size_ext = data.dims[1].dyn_size_ext  # one output frame per input frame
    ctx.mark_as_default_output(tensor=out)
'''

_FAKE_RASR_TRAINER = '''
import sys
import numpy
sys.path.insert(0, @ROOT@)
from returnn_b200.sprint import interface

action, config_file = sys.argv[1], sys.argv[2]
segments = ["corpus/seg%02i" % i for i in range(12)]


def extract(name):  # features [D, T] and an alignment that is a function of the features
    rng = numpy.random.RandomState(sum(ord(c) for c in name))
    x = rng.randn(5, 6 + int(name[-2:]) % 5).astype("float32")
    return x, numpy.argmax(x[:3], axis=0).astype("int32")


if action == "train":
    first = True
    seen = []
    for seg in interface.getSegmentList("corpus", segments, config=config_file):
        x, ali = extract(seg)
        if first:  # RASR initialises its trainer lazily, with the first data
            interface.init(inputDim=5, outputDim=3, config="action:train,configfile:" + config_file, targetMode="target-alignment")
            first = False
        interface.feedInputAndTargetAlignment(x, ali, segmentName=seg)
        seen.append(seg)
    interface.exit()
    assert len(seen) == 3 * len(segments) and sorted(seen[:12]) == segments and seen[:12] != seen[12:24], seen
    print("TRAINED", len(seen))
elif action == "forward":
    interface.init(inputDim=5, outputDim=3, config="action:forward,epoch:3,configfile:" + config_file, targetMode="forward-only")
    right = total = 0
    for seg in segments:
        x, ali = extract(seg)
        post = interface.feedInput(x, segmentName=seg)
        assert post.shape == (3, x.shape[1]) and numpy.allclose(post.sum(0), 1.0, atol=1e-4)
        right += int((post.argmax(0) == ali).sum())
        total += len(ali)
    interface.exit()
    print("FORWARDED acc %.3f" % (right / total))
else:
    scorer = interface.init(sprint_unit="PythonFeatureScorer", config="epoch:3,prior_file:%s,prior_scale:0.5,configfile:%s" % (sys.argv[3], config_file),
                            version_number=1, callback=None)
    scorer.init(5, 3)
    x, ali = extract(segments[0])
    for t in range(x.shape[1]):
        scorer.add_feature(x[:, t], t)
    scorer.compute(x.shape[1])
    s = numpy.stack([scorer.get_scores(t) for t in range(x.shape[1])], axis=1)
    post = scorer.get_posteriors()
    want = -numpy.log(post) + 0.5 * numpy.log(numpy.array([0.5, 0.25, 0.25], "float32"))[:, None]
    assert numpy.allclose(s, want, atol=1e-5), (s, want)
    scorer.reset(x.shape[1])
    scorer.exit()
    print("SCORED", s.shape)
'''


def test_interface_inside_a_stand_in_rasr_process(tmp_path):
    """segment order + trainer fed by the stand-in's corpus loop for three epochs; then forwarding and the feature scorer from the checkpoint"""
    import subprocess

    cfg = tmp_path / "returnn.config"
    cfg.write_text("#!rnn.py\n" + _INTERFACE_CONFIG.replace("@MODEL@", str(tmp_path / "net")))
    script = tmp_path / "fake_rasr.py"
    script.write_text(_FAKE_RASR_TRAINER.replace("@ROOT@", repr(_ROOT)))
    (tmp_path / "priors.txt").write_text("0.5 0.25 0.25\n")

    def run(*args):
        res = subprocess.run([sys.executable, str(script)] + list(args), capture_output=True, text=True, timeout=400, cwd=str(tmp_path))
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
        return res.stdout

    assert "TRAINED 36" in run("train", str(cfg))
    assert (tmp_path / "net.003.pt").exists()
    out = run("forward", str(cfg))
    acc = float(out.split("FORWARDED acc ")[1].split()[0])
    assert acc > 0.6, out  # three epochs of a linear model on a linearly separable rule
    assert "SCORED (3, " in run("score", str(cfg), str(tmp_path / "priors.txt"))
