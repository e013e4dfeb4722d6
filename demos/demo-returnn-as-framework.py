#!/usr/bin/env python3
"""
Use the framework as a library: build the config in Python, create datasets and the engine, train, then query the model.
"""

import _setup_env  # noqa: F401
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
        self.hidden = Dim(32, name="hidden")
        self.l1 = rf.Linear(in_dim, self.hidden)
        self.l2 = rf.Linear(self.hidden, out_dim)

    def __call__(self, x):
        return self.l2(rf.tanh(self.l1(x)))


def train_step(*, model, extern_data, **_):
    logits = model(extern_data["data"])
    rf.cross_entropy(estimated=logits, estimated_type="logits", target=extern_data["classes"], axis=out_dim).mark_as_loss("ce")


def main():
    config = Config({
        "backend": "torch", "task": "train", "num_epochs": 2, "batch_size": 2000, "optimizer": {"class": "adam"}, "learning_rate": 0.01,
        "extern_data": {"data": {"dims": (batch_dim, time_dim, in_dim), "dtype": "float32"},
                        "classes": {"dims": (batch_dim, time_dim), "sparse_dim": out_dim, "dtype": "int32"}},
        "get_model": lambda **_: Model(), "train_step": train_step, "log_verbosity": 3, "device": "cpu",
    })
    set_global_config(config)
    log.init_by_config(config)
    train = init_dataset({"class": "Task12AXDataset", "num_seqs": 200})
    dev = init_dataset({"class": "Task12AXDataset", "num_seqs": 20, "fixed_random_seed": 1})
    engine = Engine(config)
    engine.init_train_from_config(config, train, dev, None)
    engine.train()
    print("final dev scores:", engine.learning_rate_control.epoch_data[engine.epoch].error)


if __name__ == "__main__":
    main()
