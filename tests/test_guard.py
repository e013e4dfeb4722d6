"""The canary allocator of ops/guard.py itself (CPU): guards are placed, an out-of-bounds write is reported, clean code passes."""

import pytest
import torch
from returnn_b200.ops import guard


def test_canaries_detect_out_of_bounds_write_and_pass_clean_code():
    with guard.CanaryAllocations(devices=("cpu",)) as g:
        a = torch.empty(5, 7, dtype=torch.float32, device="cpu")
        b = torch.zeros((3,), dtype=torch.int32, device="cpu")
        c = torch.empty_like(a)
        d = torch.full((4,), 2.5, device="cpu")
        e = torch.empty(3, 3)  # no device given: left alone
        a.fill_(1.0)
        c.copy_(a)
    assert g.num_guarded() == 4 and a.shape == (5, 7) and a.is_contiguous() and a.data_ptr() % 64 == 0
    assert float(b.sum()) == 0 and float(d.sum()) == 10.0 and torch.equal(a, c) and e.shape == (3, 3)
    g.check()
    assert torch.empty is guard.torch.empty and "CanaryAllocations" not in repr(torch.empty)
    # a "kernel" that writes two elements past the end of b and one before the start of d
    with guard.CanaryAllocations(devices=("cpu",)) as g:
        b = torch.zeros(3, dtype=torch.int32, device="cpu")
        d = torch.zeros(4, dtype=torch.float32, device="cpu")
        torch.as_strided(b, (5,), (1,)).fill_(7)
        torch.as_strided(d, (1,), (1,), storage_offset=d.storage_offset() - 1).fill_(1.0)
    bad = g.violations()
    assert len(bad) == 2 and "after the tensor" in bad[0] and "offset 12" in bad[0] and "before the tensor" in bad[1], bad
    with pytest.raises(guard.GuardViolation):
        g.check()


def test_check_repeatable_flags_nondeterminism():
    x = torch.arange(6.0)
    guard.check_repeatable(lambda: (x * 2, [x + 1]))
    state = {"n": 0}

    def flaky():
        state["n"] += 1
        return x + state["n"]

    with pytest.raises(AssertionError):
        guard.check_repeatable(flaky)
