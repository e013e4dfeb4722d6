"""whole-step CUDA-graph replay (config option torch_cuda_graph) gives the same training trajectory as the eager engine"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _train(graph: bool, tmp_path):
    from returnn_b200.config import Config, set_global_config
    from returnn_b200.log import log
    from returnn_b200.datasets.basic import init_dataset
    from returnn_b200.torch.engine import Engine
    from returnn_b200.tensor import Dim, batch_dim
    import returnn_b200.frontend as rf

    time_dim, in_dim, out_dim = Dim(None, name="time"), Dim(9, name="in"), Dim(2, name="out")

    class Model(rf.Module):
        def __init__(self):
            super().__init__()
            self.hidden = Dim(64, name="hidden")
            self.l1 = rf.Linear(in_dim, self.hidden)
            self.l2 = rf.Linear(self.hidden, out_dim)

        def __call__(self, x):
            return self.l2(rf.relu(self.l1(x)))

    def train_step(*, model, extern_data, **_):
        logits = model(extern_data["data"])
        rf.cross_entropy(estimated=logits, estimated_type="logits", target=extern_data["classes"], axis=out_dim).mark_as_loss("ce")

    opts = {
        "backend": "torch", "task": "train", "num_epochs": 2, "batch_size": 1500, "max_seqs": 20, "optimizer": {"class": "adam"}, "learning_rate": 0.01,
        "device": "cuda", "log_verbosity": 2, "random_seed": 7,
        "extern_data": {"data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"},
                        "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32"}},
        "get_model": lambda **_: Model(), "train_step": train_step,
    }
    if graph:
        opts["torch_cuda_graph"] = {"batch_size_bound": 20, "dim_capacity": {"data": 110, "classes": 110}, "warmup_steps": 2}
    config = Config(opts)
    set_global_config(config)
    log.init_by_config(config)
    torch.manual_seed(7)
    train = init_dataset({"class": "Task12AXDataset", "num_seqs": 200, "fixed_random_seed": 3})
    dev = init_dataset({"class": "Task12AXDataset", "num_seqs": 30, "fixed_random_seed": 1})
    engine = Engine(config)
    engine.init_train_from_config(config, train, dev, None)
    engine.train()
    scores = engine.learning_rate_control.epoch_data[engine.epoch].error
    params = {k: v.detach().float().cpu().clone() for k, v in engine.get_pt_model().state_dict().items()}
    return scores, params


def test_graph_replay_matches_eager(tmp_path):
    s_eager, p_eager = _train(False, tmp_path)
    s_graph, p_graph = _train(True, tmp_path)
    assert abs(s_eager["train_loss_ce"] - s_graph["train_loss_ce"]) < 2e-3, (s_eager, s_graph)
    assert abs(s_eager["dev_loss_ce"] - s_graph["dev_loss_ce"]) < 2e-3, (s_eager, s_graph)
    for k in p_eager:
        torch.testing.assert_close(p_graph[k], p_eager[k], atol=2e-3, rtol=2e-2)
