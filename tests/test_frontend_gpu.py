"""Implicit-GEMM conv subsampling frontend against the torch (cuDNN / fp32) path: packed outputs and all parameter gradients."""

import pytest
import torch

gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("lens", [[100, 57, 98, 3], [301, 300, 299]])
def test_frontend_native_matches_torch_path(lens):
    from returnn_b200.tensor import Dim
    from returnn_b200.frontend.encoder.conformer import ConformerEncoder, ConformerConvSubsample
    from returnn_b200.torch.frontend.bridge import rf_module_to_pt_module
    from returnn_b200.models import conformer_fused
    from returnn_b200.models.packing import PackInfo
    from returnn_b200.utils.basic import BehaviorVersion

    BehaviorVersion._reset(24)
    torch.manual_seed(0)
    f = Dim(80, name="feat")
    enc = ConformerEncoder(f, Dim(64, name="model"), num_layers=1, num_heads=1, ff_dim=Dim(64, name="ff"), conv_kernel_size=3, dropout=0.0, att_dropout=0.0,
                           input_layer=ConformerConvSubsample(f, out_dims=[Dim(32, name="c1"), Dim(64, name="c2"), Dim(64, name="c3")],
                                                              filter_sizes=[(3, 3), (3, 3), (3, 3)], pool_sizes=[(1, 2)], strides=[(1, 1), (3, 1), (2, 1)]))
    pt = rf_module_to_pt_module(enc).to("cuda")
    with torch.no_grad():
        for n, p in pt.named_parameters():
            if "input_layer" in n and p.dim() == 1:
                p.normal_(0.0, 0.2)
    lens_host = torch.tensor(lens, dtype=torch.int32)
    feats = torch.randn(len(lens), max(lens), 80, device="cuda")
    params = [p for n, p in pt.named_parameters() if "input_layer" in n]
    # native
    x, pack = conformer_fused._frontend_native(enc, feats, lens_host)
    assert x is not None
    wgt = torch.randn_like(x.float())
    (x.float() * wgt).sum().backward()
    g_native = [p.grad.clone() for p in params]
    for p in params:
        p.grad = None
    # torch path in fp32
    W = conformer_fused._Weights(torch.float32)
    x_pad, lens2 = conformer_fused.frontend_subsample(enc, feats, lens_host, W)
    pack2 = PackInfo(lens2, feats.device, padded_len=x_pad.shape[1])
    ref = pack2.pack(x_pad)
    assert ref.shape == x.shape and pack2.lens_host.tolist() == pack.lens_host.tolist()
    (ref * wgt).sum().backward()
    torch.testing.assert_close(x.float(), ref, atol=0.06, rtol=0.05)
    errs = {}
    for p, g, (n, _) in zip(params, g_native, [(n, p) for n, p in pt.named_parameters() if "input_layer" in n]):
        scale = float(p.grad.abs().max()) + 1e-6
        errs[n] = (float((g.float() - p.grad).abs().max()) / scale, float(torch.nn.functional.cosine_similarity(g.float().flatten(), p.grad.flatten(), dim=0)))
    # bf16 activations and gradients through three layers against an fp32 reference: direction must agree closely, magnitudes within 10 %
    assert all(e < 0.1 and c > 0.995 for e, c in errs.values()), errs
