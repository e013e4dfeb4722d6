"""
Packed execution of plain RF models (returnn_b200/frontend/packed_mode.py): a Conformer encoder built from the ordinary RF modules gives
the same outputs and parameter gradients whether its layers run on padded [batch, time, model] tensors or on the packed valid frames.
"""

import numpy
import pytest
import torch

import returnn_b200.frontend as rf
from returnn_b200.tensor import Tensor, Dim, batch_dim
from returnn_b200.frontend import packed_mode

gpu = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _behavior():
    from returnn_b200.utils.basic import BehaviorVersion

    BehaviorVersion._reset(24)
    yield
    BehaviorVersion._reset()


def _time_dim(lens):
    batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(len(lens), dtype=torch.int32))
    d = Dim(None, name="time")
    d.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor(lens, dtype=torch.int32))
    return d


def test_pack_unpack_round_trip_and_op_dispatch():
    torch.manual_seed(0)
    lens = [7, 3, 5]
    time = _time_dim(lens)
    feat = Dim(4, name="feat")
    raw = torch.randn(3, 7, 4)
    for b, n in enumerate(lens):
        raw[b, n:] = 0
    x = Tensor("x", dims=[batch_dim, time, feat], dtype="float32", raw_tensor=raw)
    p = packed_mode.pack_padded_tensor(x, dims=(batch_dim, time))
    assert p.raw_tensor.shape == (15, 4) and packed_mode.packed_dim_of(p, time) is p.dims[0] and packed_mode.packed_dim_of(x, time) is None
    assert torch.equal(p.raw_tensor[7:10], raw[1, :3])
    back = packed_mode.unpack_to_padded(p)
    assert back.dims == (batch_dim, time, feat) and torch.equal(back.raw_tensor, raw)
    # an op along time on packed rows: depthwise conv with "same" padding keeps the time dim, a strided pool makes a new one
    rf.init_train_step_run_ctx(train_flag=False, step=0, epoch=1)
    conv = rf.Conv1d(feat, feat, filter_size=3, groups=4, padding="same")
    y_pad, _ = conv(x, in_spatial_dim=time)
    y_packed, out_dims = conv(p, in_spatial_dim=time)
    assert y_packed.dims[0] is p.dims[0]
    got = packed_mode.unpack_to_padded(y_packed).raw_tensor
    ref = y_pad.copy_transpose([batch_dim, time, feat]).raw_tensor
    for b, n in enumerate(lens):
        assert torch.allclose(got[b, :n], ref[b, :n], atol=1e-6)
    z_pad, zt = rf.pool1d(x, mode="max", pool_size=2, padding="same", in_spatial_dim=time)
    z_packed, zt2 = rf.pool1d(p, mode="max", pool_size=2, padding="same", in_spatial_dim=time)
    new_p = z_packed.dims[0]
    assert new_p is not p.dims[0] and new_p.packed_info.pack.lens_host.tolist() == [4, 2, 3]


def _build_encoder():
    from returnn_b200.frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample

    in_dim, model = Dim(10, name="in"), Dim(16, name="model")
    rf.set_random_seed(3)
    torch.manual_seed(3)
    enc = ConformerEncoder(
        in_dim, model, num_layers=2, num_heads=2, ff_dim=Dim(32, name="ff"), conv_kernel_size=5, dropout=0.0, att_dropout=0.0, input_dropout=0.0,
        conv_norm=rf.build_dict(rf.BatchNorm, use_mask=True),  # statistics over valid frames only, which is what packed rows are
        input_layer=ConformerConvSubsample(in_dim, out_dims=[Dim(3, name="c1"), Dim(4, name="c2")], filter_sizes=[(3, 3), (3, 3)], pool_sizes=[(1, 2)],
                                           strides=[(1, 1), (2, 1)]))
    return enc, in_dim, model


def _run(enc, in_dim, model, dev, packed: bool, train: bool):
    lens = [23, 11, 17]
    time = _time_dim(lens)
    torch.manual_seed(5)
    raw = torch.randn(3, 23, 10)
    for b, n in enumerate(lens):
        raw[b, n:] = 0
    x = Tensor("x", dims=[batch_dim, time, in_dim], dtype="float32", raw_tensor=raw.to(dev))
    rf.init_train_step_run_ctx(train_flag=train, step=0, epoch=1)
    for p in enc.parameters():
        p.raw_tensor.grad = None
    with packed_mode.packed_mode_ctx(packed):
        y, out_time = enc(x, in_spatial_dim=time)
    out = y.copy_transpose([batch_dim, out_time, model]).raw_tensor
    out_lens = out_time.dyn_size_ext.raw_tensor.tolist()
    mask = (torch.arange(out.shape[1])[None, :] < torch.tensor(out_lens)[:, None]).to(out.device)
    weights = torch.linspace(0.5, 1.5, out.numel(), device=out.device).reshape(out.shape)
    ((out * weights) * mask[:, :, None]).sum().backward()
    grads = {name: p.raw_tensor.grad.detach().clone() for name, p in enc.named_parameters() if p.raw_tensor.grad is not None}
    return (out * mask[:, :, None]).detach(), grads


@pytest.mark.parametrize("train", [False, True])
def test_plain_rf_conformer_packed_equals_padded_cpu(train):
    enc, in_dim, model = _build_encoder()
    out_pad, g_pad = _run(enc, in_dim, model, "cpu", packed=False, train=train)
    out_packed, g_packed = _run(enc, in_dim, model, "cpu", packed=True, train=train)
    assert out_pad.shape == out_packed.shape
    assert torch.allclose(out_pad, out_packed, atol=2e-5), float((out_pad - out_packed).abs().max())
    assert set(g_pad) == set(g_packed) and len(g_pad) > 40
    for name in g_pad:
        assert torch.allclose(g_pad[name], g_packed[name], atol=2e-4, rtol=1e-3), (name, float((g_pad[name] - g_packed[name]).abs().max()))


@gpu
def test_plain_rf_conformer_packed_equals_padded_gpu():
    """on the GPU the packed layers run the varlen attention kernels"""
    enc, in_dim, model = _build_encoder()
    for p in enc.parameters():
        p.raw_tensor.data = p.raw_tensor.data.cuda()
    for name in ("running_mean", "running_variance"):
        for layer in enc.layers:
            norm = layer.conv_block.norm
            if hasattr(norm, name):
                getattr(norm, name).raw_tensor = getattr(norm, name).raw_tensor.cuda()
    out_pad, g_pad = _run(enc, in_dim, model, "cuda", packed=False, train=False)
    out_packed, g_packed = _run(enc, in_dim, model, "cuda", packed=True, train=False)
    assert torch.allclose(out_pad, out_packed, atol=2e-2), float((out_pad - out_packed).abs().max())


def test_packed_regap_and_flat_content():
    """re-layout of a packed tensor with gaps and aligned starts, and the dense flat view: same sequences, zeros in between"""
    import torch
    import returnn_b200.frontend as rf
    from returnn_b200.tensor import Tensor, Dim, batch_dim

    lens = [3, 1, 4]
    t = Dim(None, name="time")
    batch_dim.dyn_size_ext = Tensor("batch_size", dims=[], dtype="int32", raw_tensor=torch.tensor(3, dtype=torch.int32))
    t.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor(lens, dtype=torch.int32))
    f = Dim(2, name="f")
    raw = torch.arange(3 * 4 * 2, dtype=torch.float32).reshape(3, 4, 2) + 1.0
    x = Tensor("x", dims=[batch_dim, t, f], dtype="float32", raw_tensor=raw, feature_dim=f)
    p = rf.pack(x, dims=[batch_dim, t])
    assert p.gap == 0 and p.align == 1 and p.raw_tensor.shape[0] == 8
    g = rf.packed_regap(p, 2, align=4)
    # starts: 0, then 3 + 2 = 5 -> aligned to 8, then 8 + 1 + 2 = 11 -> 12; end 12 + 4 + 2 = 18
    assert g.seq_starts.tolist() == [0, 8, 12] and g.raw_tensor.shape[0] == 18 and (g.gap, g.align) == (2, 4)
    for b, (s, n) in enumerate(zip([0, 8, 12], lens)):
        torch.testing.assert_close(g.raw_tensor[s: s + n], raw[b, :n])
    holes = torch.ones(18, dtype=torch.bool)
    for s, n in zip([0, 8, 12], lens):
        holes[s: s + n] = False
    assert float(g.raw_tensor[holes].abs().max()) == 0.0
    assert rf.packed_regap(g, 2, align=4) is g
    b24 = rf.packed_regap(p, 1, total_bound=24)
    assert b24.raw_tensor.shape[0] == 24 and b24.packed_dim.capacity == 24 and float(b24.raw_tensor[11:].abs().max()) == 0.0
    flat, flat_dim = rf.packed_flat_content(g)
    assert flat.dims == (flat_dim, f) and int(flat_dim.dyn_size_ext.raw_tensor) == 8
    torch.testing.assert_close(flat.raw_tensor, p.raw_tensor)
    back = rf.unpack(g)
    torch.testing.assert_close(back.raw_tensor, x.copy_masked(0.0).raw_tensor)
