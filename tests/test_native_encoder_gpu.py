"""
Native Conformer encoder executor (one call per pass) against the per-op path on the same weights: outputs, input
gradient and all parameter gradients, without dropout; with dropout: reproducible for a fixed RNG state and finite.
"""

import pytest
import torch

gpu = pytest.mark.gpu


def _make(num_layers=2, model_dim=128, heads=2, ff=256, conv_k=7, dropout=0.0):
    from returnn_b200.tensor import Dim
    from returnn_b200.models.conformer_ctc import ConformerCtcModel
    from returnn_b200.torch.frontend.bridge import rf_module_to_pt_module
    from returnn_b200.parallel.arena import ParamArena
    from returnn_b200.utils.basic import BehaviorVersion

    BehaviorVersion._reset(24)  # convolutions mask padded input: the semantics of the fused path
    torch.manual_seed(1)
    model = ConformerCtcModel(in_dim=Dim(80, name="feat"), vocab_dim=Dim(55, name="vocab"), num_layers=num_layers, model_dim=model_dim,
                              num_heads=heads, ff_dim=ff, conv_kernel_size=conv_k, dropout=dropout, att_dropout=dropout,
                              conv_channels=(8, 16, 16))
    pt = rf_module_to_pt_module(model).to("cuda")
    with torch.no_grad():
        for n, p in pt.named_parameters():
            if p.dim() == 1 and ("bias" in n or "beta" in n):
                p.normal_(0.0, 0.1)  # biases are zero-initialised: give them values so that their paths are exercised
    arena = ParamArena(list(pt.named_parameters()))
    return model, pt, arena


def _run(model, arena, feats, lens, wgt, native: bool):
    from returnn_b200.models import conformer_fused, conformer_native
    from returnn_b200.ops.elementwise import _seed_tensor

    conformer_native.ENABLED = native
    seed = _seed_tensor(feats.device)
    seed[0] = 777
    seed[1] = 0
    arena.zero_grad()
    f = feats.clone().requires_grad_(True)
    out, pack = conformer_fused.encode_packed(model.encoder, f, lens, training=True)
    loss = (out.float() * wgt[: out.shape[0]]).sum()
    loss.backward()
    arena.relink_grads()
    conformer_native.ENABLED = True
    # the features are data: the conv frontend returns no gradient for them; the frontend's own parameters are part of the arena
    return out.detach().float(), None, arena.flat_grad.clone()


@gpu
def test_native_encoder_matches_per_op_path():
    from returnn_b200.models import conformer_fused, conformer_native

    model, pt, arena = _make()
    assert conformer_fused.supports_fused(model.encoder)
    assert conformer_native.get_plan(model.encoder) is not None
    torch.manual_seed(2)
    lens = torch.tensor([600, 431, 577, 90], dtype=torch.int32)
    feats = torch.randn(4, 600, 80, device="cuda")
    wgt = torch.randn(600, 128, device="cuda")
    o1, gx1, gp1 = _run(model, arena, feats, lens, wgt, native=True)
    o2, gx2, gp2 = _run(model, arena, feats, lens, wgt, native=False)
    assert torch.isfinite(o1).all() and torch.isfinite(gp1).all()
    torch.testing.assert_close(o1, o2, atol=0.08, rtol=0.05)
    # gradients: compare per parameter relative to the parameter's gradient scale (bf16 paths differ in rounding order)
    bad = []
    for s in arena.slots:
        if s.name.endswith("depthwise_conv.bias"):
            continue  # a bias in front of BatchNorm has an exactly zero gradient: both paths only produce rounding noise
        a, b = gp1[s.offset: s.offset + s.numel], gp2[s.offset: s.offset + s.numel]
        scale = float(b.abs().max()) + 1e-6
        err = float((a - b).abs().max()) / scale
        if err >= 0.08:
            bad.append("%s: rel. max err %.4f (scale %.3g)" % (s.name, err, scale))
    assert not bad, "parameter gradients differ:\n" + "\n".join(bad)


@gpu
def test_native_encoder_dropout_reproducible():
    from returnn_b200.models import conformer_native

    model, pt, arena = _make(dropout=0.1)
    assert conformer_native.get_plan(model.encoder) is not None
    torch.manual_seed(3)
    lens = torch.tensor([300, 256], dtype=torch.int32)
    feats = torch.randn(2, 300, 80, device="cuda")
    wgt = torch.randn(300, 128, device="cuda")
    o1, gx1, gp1 = _run(model, arena, feats, lens, wgt, native=True)
    o2, gx2, gp2 = _run(model, arena, feats, lens, wgt, native=True)
    assert torch.isfinite(o1).all() and torch.isfinite(gp1).all()
    torch.testing.assert_close(o1, o2, atol=0.0, rtol=0.0)
    # atomics make the weight gradients order-dependent in the last bits only
    torch.testing.assert_close(gp1, gp2, atol=1e-2, rtol=1e-2)
    from returnn_b200.ops import gemm

    gemm.check_status()


@gpu
def test_native_encoder_stays_inside_its_workspace():
    """forward + backward of the executor with canary regions around its workspace and every tensor of the fused path"""
    from returnn_b200.ops import guard, gemm

    model, pt, arena = _make(dropout=0.1)
    torch.manual_seed(3)
    for lens in (torch.tensor([600, 431, 577, 90], dtype=torch.int32), torch.tensor([61], dtype=torch.int32), torch.tensor([333, 1999, 64], dtype=torch.int32)):
        feats = torch.randn(len(lens), int(lens.max()), 80, device="cuda")
        wgt = torch.randn(int((lens // 6 + 2).sum()), model.model_dim.dimension, device="cuda")
        with guard.CanaryAllocations() as g:
            out, _, grads = _run(model, arena, feats, lens, wgt, native=True)
        g.check()
        gemm.check_status()
        assert g.num_guarded() > 0 and bool(torch.isfinite(out).all()) and bool(torch.isfinite(grads).all())


@gpu
def test_native_encoder_against_fp32_rf_oracle():
    """
    The native executor (bf16, own kernels, packed rows) against an independent oracle: the SAME module called through the ordinary
    RF path (``ConformerEncoder.__call__`` on padded tensors) on the CPU in fp32, where no kernel of this repository runs.
    Outputs and every parameter gradient, relative to their scale, at bf16 tolerances.
    """
    import copy
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Tensor, Dim, batch_dim
    from returnn_b200.models import conformer_fused, conformer_native

    from returnn_b200.utils.basic import BehaviorVersion

    model, pt, arena = _make()
    BehaviorVersion._reset(24)  # convolutions mask their padded input (default from 23): what the executor computes on valid frames
    model.encoder.input_dropout = 0.0  # the RF path draws its dropout from torch's generator, the executor from its counter-based one
    torch.manual_seed(2)
    lens = torch.tensor([600, 431, 577, 90], dtype=torch.int32)
    feats = torch.randn(4, 600, 80, device="cuda")
    for b, n in enumerate(lens.tolist()):
        feats[b, n:] = 0
    wgt = torch.randn(600, 128, device="cuda")
    out_native, _, grads_native = _run(model, arena, feats, lens, wgt, native=True)
    # the oracle: a CPU fp32 copy of the module tree, RF call on padded [B, T, F]
    state = {k: v.detach().float().cpu().clone() for k, v in pt.state_dict().items()}
    cpu_model = copy.deepcopy(model)
    assert all(layer.conv_block.norm.use_mask for layer in cpu_model.encoder.layers)  # BatchNorm statistics over valid frames
    from returnn_b200.torch.frontend.bridge import rf_module_to_pt_module

    cpu_pt = rf_module_to_pt_module(cpu_model).to("cpu").float()
    cpu_pt.load_state_dict(state)
    rf.init_train_step_run_ctx(train_flag=True, step=0, epoch=1)
    batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(4, dtype=torch.int32))
    time = Dim(None, name="time")
    time.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=lens.clone())
    enc = cpu_model.encoder
    x = Tensor("x", dims=[batch_dim, time, enc.in_dim], dtype="float32", raw_tensor=feats.cpu())
    y, out_time = enc(x, in_spatial_dim=time)
    y_raw = y.copy_transpose([batch_dim, out_time, enc.out_dim]).raw_tensor
    out_lens = out_time.dyn_size_ext.raw_tensor.tolist()
    rows = torch.cat([y_raw[b, : int(n)] for b, n in enumerate(out_lens)])  # the packed order of the executor's output
    assert rows.shape == out_native.shape
    (rows * wgt.cpu()[: rows.shape[0]]).sum().backward()
    scale = float(rows.detach().abs().max())
    err = float((out_native.cpu() - rows.detach()).abs().max()) / scale
    assert err < 0.05, "outputs: rel. max err %.4f" % err
    cpu_grads = {n: p.grad for n, p in cpu_pt.named_parameters()}
    bad = []
    for s in arena.slots:
        if s.name.endswith("depthwise_conv.bias"):
            continue  # in front of BatchNorm: exactly zero gradient, only rounding noise on both sides
        g_ref = cpu_grads.get(s.name)
        if g_ref is None:
            continue
        a = grads_native[s.offset: s.offset + s.numel].cpu()
        b_ = g_ref.reshape(-1)
        sc = float(b_.abs().max()) + 1e-6
        e = float((a - b_).abs().max()) / sc
        # The conv frontend sums its filter / bias gradients over every frame and frequency of the batch, with heavy cancellation: bf16
        # activations alone (plain torch, same arithmetic) move them by 5-11 % of their maximum against fp32, so direction is the
        # criterion there and the magnitude bound is wider.
        if "input_layer" in s.name:
            cos = float(torch.nn.functional.cosine_similarity(a.double(), b_.double(), dim=0))
            if e >= 0.25 or cos < 0.99:
                bad.append("%s: rel. max err %.4f, cosine %.4f (scale %.3g)" % (s.name, e, cos, sc))
        elif e >= 0.1:
            bad.append("%s: rel. max err %.4f (scale %.3g)" % (s.name, e, sc))
    assert not bad, "parameter gradients differ from the fp32 oracle:\n" + "\n".join(bad)
