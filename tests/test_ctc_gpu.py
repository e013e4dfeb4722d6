"""
Fused CTC kernels (log-softmax + alpha/beta + gradient on packed logits) against torch.nn.functional.ctc_loss in fp32.
"""

import pytest
import torch

gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("lens,tlens,V,dtype", [
    ([30, 22, 5], [7, 3, 2], 50, torch.float32),
    ([334, 200, 120, 60], [11, 7, 4, 2], 10001, torch.bfloat16),
    ([12, 9], [4, 9], 33, torch.float32),       # second sequence: 9 labels in 9 frames (feasible only without repeats)
    ([6, 3], [2, 5], 17, torch.float32),        # second sequence infeasible -> loss 0, zero grad
    ([40], [0], 20, torch.float32),             # empty target
])
def test_ctc_loss_packed(lens, tlens, V, dtype):
    from returnn_b200.models.packing import PackInfo
    from returnn_b200.ops import ctc, _lib

    torch.manual_seed(0)
    B = len(lens)
    pack = PackInfo(torch.tensor(lens, dtype=torch.int32), torch.device("cuda"))
    blank = V - 1
    S = max(max(tlens), 1)
    targets = torch.randint(0, V - 1, (B, S), device="cuda", dtype=torch.int32)
    if len(lens) == 2 and tlens[1] == 9:
        targets[1] = torch.arange(9, device="cuda", dtype=torch.int32)  # no repeats
    tl = torch.tensor(tlens, dtype=torch.int32)
    logits = (torch.randn(pack.n, V, device="cuda") * 2).to(dtype).requires_grad_(True)
    w = torch.rand(B, device="cuda") + 0.5
    n0 = _lib.launch_count()
    loss = ctc.ctc_loss_packed(logits, pack, targets, tl, blank_index=blank)
    assert _lib.launch_count() > n0, "native kernels did not run"
    (loss * w).sum().backward()
    l32 = logits.detach().float().requires_grad_(True)
    padded = pack.unpack(l32)
    lp = torch.log_softmax(padded, dim=-1).transpose(0, 1)
    ref = torch.nn.functional.ctc_loss(lp, targets.long(), pack.lens_host.long(), tl.long(), blank=blank, reduction="none", zero_infinity=True)
    (ref * w).sum().backward()
    tol = 5e-2 if dtype == torch.bfloat16 else 1e-3
    torch.testing.assert_close(loss, ref, atol=tol, rtol=1e-3)
    gtol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(logits.grad.float(), l32.grad, atol=gtol, rtol=1e-2)
