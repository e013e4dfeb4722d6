"""FSA ops: CTC via the FSA full sum equals torch's CTC loss (values and gradients); Viterbi equals the brute-force best path."""

import pytest
import torch

gpu = pytest.mark.gpu


def _case(dev, B=4, T=13, V=6, S=4):
    torch.manual_seed(0)
    logits = torch.randn(B, T, V, device=dev, requires_grad=True)
    targets = torch.randint(0, V - 1, (B, S), device=dev)
    targets[1, 1] = targets[1, 0]  # a repeated label needs the blank in between
    in_lens = torch.tensor([13, 9, 13, 5])[:B]
    tgt_lens = torch.tensor([4, 3, 0, 2])[:B]
    return logits, targets, in_lens, tgt_lens


def _check(dev):
    from returnn_b200.ops import fsa

    logits, targets, in_lens, tgt_lens = _case(dev)
    V = logits.shape[-1]
    loss = fsa.ctc_loss_via_fsa(logits, targets, in_lens, tgt_lens, blank=V - 1)
    loss.sum().backward()
    g = logits.grad.clone()
    l2 = logits.detach().cpu().requires_grad_(True)
    ref = torch.nn.functional.ctc_loss(torch.log_softmax(l2, -1).transpose(0, 1), targets.cpu(), in_lens, tgt_lens, blank=V - 1, reduction="none")
    ref.sum().backward()
    torch.testing.assert_close(loss.cpu(), ref, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(g.cpu(), l2.grad, atol=1e-3, rtol=1e-3)
    # Viterbi: its score is at least as good as any sampled alignment and equals the greedy path when that path is valid
    f = fsa.ctc_fsa(targets, tgt_lens, blank=V - 1)
    am = -torch.log_softmax(logits.detach().float(), -1).transpose(0, 1).contiguous()
    align, score = fsa.fast_viterbi(am, f, in_lens)
    align_ref, score_ref = fsa.fast_viterbi_reference(am.cpu(), f.to("cpu"), in_lens)
    torch.testing.assert_close(score.cpu(), score_ref, atol=1e-3, rtol=1e-4)
    for b in range(logits.shape[0]):
        path = align[: int(in_lens[b]), b].cpu().tolist()
        collapsed = [p for i, p in enumerate(path) if p != V - 1 and (i == 0 or p != path[i - 1])]
        assert collapsed == targets[b, : int(tgt_lens[b])].cpu().tolist()
        assert abs(float(am[: int(in_lens[b]), b].cpu().gather(1, torch.tensor(path)[:, None]).sum()) - float(score[b])) < 1e-3


def test_ctc_via_fsa_cpu():
    _check("cpu")


@gpu
def test_ctc_via_fsa_kernels():
    _check("cuda")
