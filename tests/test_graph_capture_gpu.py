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


@pytest.mark.gpu
def test_graphed_decoder_loss_equals_eager():
    """decoder + label-smoothed CE as a captured forward / backward graph pair: loss, error count, gradient into the encoder output and parameter gradients
    equal the eager formulation, for two different batches through the same graphs (and a batch beyond the bounds is refused)"""
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Tensor, Dim, batch_dim
    from returnn_b200.frontend.decoder.transformer import TransformerDecoder
    from returnn_b200.models.graphed_decoder import GraphedDecoderLoss
    from returnn_b200.torch.frontend.bridge import rf_module_to_pt_module
    from returnn_b200.utils.basic import BehaviorVersion

    BehaviorVersion._reset(24)
    torch.manual_seed(0)
    dev = torch.device("cuda")
    vocab, enc_dim = Dim(50, name="vocab"), Dim(128, name="enc")
    dec = TransformerDecoder(encoder_dim=enc_dim, vocab_dim=vocab, model_dim=Dim(128, name="dec"), num_layers=2, num_heads=2, ff_dim=Dim(256, name="ff"),
                             dropout=0.0, att_dropout=0.0)
    pt = rf_module_to_pt_module(dec).to(dev)
    params = [p for p in pt.parameters() if p.requires_grad]
    gd = GraphedDecoderLoss(dec, vocab_dim=vocab, enc_dim=enc_dim, bos=0, eos=0, label_smoothing=0.1, batch_bound=5, enc_capacity=24, tgt_capacity=8)
    assert not gd.fits(6, 10, 4) and not gd.fits(2, 30, 4) and gd.fits(5, 24, 8)

    def eager(enc_raw, enc_lens, tgt_raw, tgt_lens):
        B = enc_raw.shape[0]
        batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(B, dtype=torch.int32))
        es, ts = Dim(None, name="enc-time"), Dim(None, name="tgt-time")
        es.dyn_size_ext = Tensor("el", dims=[batch_dim], dtype="int32", raw_tensor=enc_lens)
        ts.dyn_size_ext = Tensor("tl", dims=[batch_dim], dtype="int32", raw_tensor=tgt_lens)
        enc = Tensor("enc", dims=[batch_dim, es, enc_dim], dtype="float32", raw_tensor=enc_raw, feature_dim=enc_dim)
        tgt = Tensor("y", dims=[batch_dim, ts], dtype="int32", sparse_dim=vocab, raw_tensor=tgt_raw)
        inp, (ext,) = rf.pad(tgt, axes=[ts], padding=[(1, 0)], value=0)
        out_t, _ = rf.pad(tgt, axes=[ts], padding=[(0, 1)], value=0, out_dims=[ext], handle_dynamic_dims=True)
        logits, _ = dec(inp, spatial_dim=ext, encoder=dec.transform_encoder(enc, axis=es), state=dec.default_initial_state(batch_dims=[batch_dim]))
        ce, best = rf.softmax_cross_entropy_smoothed_grad(logits=logits, target=out_t, axis=vocab, smoothing=0.1, with_argmax=True)
        return rf.reduce_sum(ce, axis=ce.dims).raw_tensor, rf.reduce_sum(rf.cast(best != out_t, "float32"), axis=ce.dims).raw_tensor

    rf.init_train_step_run_ctx(train_flag=True, step=0, epoch=1)
    for seed, (B, T, S) in enumerate([(3, 20, 6), (5, 24, 8), (2, 9, 3)]):
        g = torch.Generator().manual_seed(seed)
        enc_lens = torch.randint(3, T + 1, (B,), generator=g, dtype=torch.int32)
        enc_lens[0] = T
        tgt_lens = torch.randint(1, S + 1, (B,), generator=g, dtype=torch.int32)
        tgt_lens[0] = S
        enc_raw = torch.randn(B, T, 128, generator=g).to(dev)
        tgt_raw = torch.randint(1, 50, (B, S), generator=g, dtype=torch.int32).to(dev)
        res = {}
        for mode in ("graph", "eager"):
            x = enc_raw.clone().requires_grad_(True)
            for p in params:
                p.grad = None
            with torch.autocast("cuda", dtype=torch.bfloat16):
                ce, wrong = (gd if mode == "graph" else eager)(x, enc_lens, tgt_raw, tgt_lens)
            ce.backward()
            res[mode] = (float(ce), float(wrong), x.grad.clone(), [p.grad.clone() if p.grad is not None else None for p in params])
        (c1, w1, gx1, gp1), (c2, w2, gx2, gp2) = res["graph"], res["eager"]
        assert abs(c1 - c2) <= 2e-3 * abs(c2) + 1e-2, (c1, c2)
        assert abs(w1 - w2) <= 1.0  # an arg-max tie in bf16 may fall either way
        scale = float(gx2.abs().max()) + 1e-9
        assert float((gx1 - gx2).abs().max()) / scale < 0.03
        for a, b in zip(gp1, gp2):
            assert (a is None) == (b is None)
            if a is not None:
                assert float((a - b).abs().max()) / (float(b.abs().max()) + 1e-9) < 0.03
    assert gd.num_replays == 3
