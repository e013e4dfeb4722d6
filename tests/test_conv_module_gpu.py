"""
Fused conv-module kernels (GLU + depthwise conv + masked BatchNorm + SiLU on packed rows) against the torch math in fp32.
"""

import pytest
import torch

gpu = pytest.mark.gpu


class _BN:
    """the attributes of rf.BatchNorm that the op reads"""

    def __init__(self, C, device):
        class P:
            def __init__(self, t):
                self.raw_tensor = t

        self.affine = True
        self.eps = 1e-3
        self.momentum = 0.1
        self.gamma = P((torch.rand(C, device=device) + 0.5).requires_grad_(True))
        self.beta = P((torch.randn(C, device=device) * 0.1).requires_grad_(True))
        self.running_mean = P(torch.zeros(C, device=device))
        self.running_variance = P(torch.ones(C, device=device))


@gpu
@pytest.mark.parametrize("lens,C,K", [([50, 7, 33], 64, 32), ([334, 100, 1, 64, 200], 512, 32), ([40, 41], 128, 31), ([10], 64, 3)])
def test_conv_module_fwd_bwd(lens, C, K):
    from returnn_b200.models.packing import PackInfo
    from returnn_b200.ops import conv_module as cm, conv_module_native as cn, _lib

    torch.manual_seed(0)
    pack = PackInfo(torch.tensor(lens, dtype=torch.int32), torch.device("cuda"))
    N = pack.n
    assert cn.supports(C, K)
    x = torch.randn(N, 2 * C, device="cuda").to(torch.bfloat16).requires_grad_(True)
    filt = (torch.randn(C, 1, K, device="cuda") * 0.2).requires_grad_(True)
    bias = (torch.randn(C, device="cuda") * 0.1).requires_grad_(True)
    bn = _BN(C, "cuda")
    dz = torch.randn(N, C, device="cuda").to(torch.bfloat16)
    n0 = _lib.launch_count()
    z = cm.glu_dwconv_bn_silu(x, filt, bias, bn, pack, training=True)
    assert _lib.launch_count() > n0, "native kernels did not run"
    z.backward(dz)
    got = [z.float(), x.grad.float(), filt.grad.clone(), bias.grad.clone(), bn.gamma.raw_tensor.grad.clone(), bn.beta.raw_tensor.grad.clone()]
    rm_native = bn.running_mean.raw_tensor.clone()
    # reference: same function with the native path disabled, in fp32
    import os

    x32 = x.detach().float().requires_grad_(True)
    f32 = filt.detach().clone().requires_grad_(True)
    b32 = bias.detach().clone().requires_grad_(True)
    bn2 = _BN(C, "cuda")
    bn2.gamma.raw_tensor = bn.gamma.raw_tensor.detach().clone().requires_grad_(True)
    bn2.beta.raw_tensor = bn.beta.raw_tensor.detach().clone().requires_grad_(True)
    os.environ["RETURNN_B200_DISABLE_NATIVE"] = "1"
    try:
        orig = cn.available
        cn.available = lambda t: False
        zr = cm.glu_dwconv_bn_silu(x32, f32, b32, bn2, pack, training=True)
    finally:
        cn.available = orig
        del os.environ["RETURNN_B200_DISABLE_NATIVE"]
    zr.backward(dz.float())
    ref = [zr, x32.grad, f32.grad, b32.grad, bn2.gamma.raw_tensor.grad, bn2.beta.raw_tensor.grad]
    names = ["z", "dx", "dfilt", "dbias", "dgamma", "dbeta"]
    scale = max(1.0, N ** 0.5)
    tols = [0.05, 0.08, 0.05 * scale, 0.05 * scale, 0.05 * scale, 0.05 * scale]
    for n, g, r, t in zip(names, got, ref, tols):
        torch.testing.assert_close(g, r.float(), atol=t, rtol=5e-2, msg=lambda s, n=n: "%s: %s" % (n, s))
    torch.testing.assert_close(rm_native, bn2.running_mean.raw_tensor, atol=1e-2, rtol=1e-2)
