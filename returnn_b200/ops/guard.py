"""
Debug harness for the native kernels: out-of-bounds writes and missing stream dependencies, found without a sanitizer.

* :class:`CanaryAllocations`: while active, every tensor that the Python wrappers allocate for a kernel (``torch.empty``,
  ``zeros``, ``empty_like``, ``zeros_like``, ``full``: outputs, saved tensors, scratch) sits between two guard regions filled
  with a byte pattern. ``check()`` synchronises and reports every guard that a kernel wrote into, with the offset of the
  first damaged byte. The guards are 4 KB on each side, so the data pointer keeps the 256-byte alignment of the allocator
  (TMA descriptors and 16-byte vector accesses behave as in production).
* :func:`check_stream_order`: runs an op on the current stream and again on a side stream whose start is delayed by a spin
  kernel while its inputs are produced late on yet another stream; a kernel launched on the wrong stream, or a wrapper
  that reads its inputs before they are ready, shows up as a difference between the two results.
* :func:`check_repeatable`: the same inputs twice, bit-wise (or to a tolerance for kernels that accumulate with atomics).

Used by ``tests/test_guard_gpu.py`` over ragged shapes of every op family; usable around any code::

    with CanaryAllocations() as guard:
        y = ops.layer_norm(x, gamma, beta)
        y.sum().backward()
    guard.check()

The reference has no counterpart (no sanitizer runs, see returnn/torch/util/native_op_code_compiler.py:99-100 for its
debug asserts); its CPU emulation of kernels as oracle corresponds to the ``*_reference`` functions next to each wrapper here.
"""

from __future__ import annotations
from typing import Any, Callable, List, Optional, Sequence, Tuple
import torch

GUARD_BYTES = 4096
PATTERN = 0xA5


class GuardViolation(AssertionError):
    """a kernel wrote outside a tensor it was given"""


def _size_from_args(args: Tuple[Any, ...]) -> Optional[Tuple[int, ...]]:
    if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
        args = tuple(args[0])
    if all(isinstance(a, int) and not isinstance(a, bool) for a in args):
        return tuple(int(a) for a in args)
    return None


class CanaryAllocations:
    """context manager: guard regions around the tensors allocated inside it (see the module docstring)"""

    _FUNCS = ("empty", "zeros", "empty_like", "zeros_like", "full")

    def __init__(self, *, devices: Sequence[str] = ("cuda",), guard_bytes: int = GUARD_BYTES):
        self.devices = tuple(devices)
        self.guard_bytes = int(guard_bytes)
        self.records: List[Tuple[torch.Tensor, int, int, str]] = []  # (byte view of the whole buffer, guard bytes, payload bytes, what)
        self._orig = {}

    # -- allocation ------------------------------------------------------------------------------------------------------
    def _guarded(self, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device, fill: Optional[float], what: str) -> torch.Tensor:
        item = dtype.itemsize
        n = 1
        for s in shape:
            n *= s
        g = self.guard_bytes
        payload = n * item
        pad = (-payload) % 256
        raw = self._orig["empty"](g + payload + pad + g, dtype=torch.uint8, device=device)
        raw[:g].fill_(PATTERN)
        raw[g + payload:].fill_(PATTERN)
        body = raw[g: g + payload].view(dtype).view(shape)
        if fill is not None:
            body.fill_(fill)
        self.records.append((raw, g, payload, "%s%s %s" % (what, list(shape), str(dtype).replace("torch.", ""))))
        return body

    def _want(self, device) -> bool:
        return torch.device(device).type in self.devices

    def _wrap(self, name: str) -> Callable:
        orig = self._orig[name]
        outer = self

        def like(t, *args, **kwargs):
            dtype = kwargs.get("dtype") or t.dtype
            device = kwargs.get("device") or t.device
            extra = set(kwargs) - {"dtype", "device"}
            if args or extra or not outer._want(device) or t.layout != torch.strided or not t.is_contiguous():
                return orig(t, *args, **kwargs)
            return outer._guarded(tuple(t.shape), dtype, torch.device(device), 0.0 if name == "zeros_like" else None, name)

        def sized(*args, **kwargs):
            fill = None
            a = args
            if name == "full":
                if len(args) != 2:
                    return orig(*args, **kwargs)
                a, fill = (args[0],), args[1]
            elif name == "zeros":
                fill = 0.0
            shape = _size_from_args(a)
            device = kwargs.get("device")
            extra = set(kwargs) - {"dtype", "device"}
            if shape is None or extra or device is None or not outer._want(device):
                return orig(*args, **kwargs)
            dtype = kwargs.get("dtype")
            if dtype is None:
                if name == "full" and isinstance(fill, bool):
                    dtype = torch.bool
                elif name == "full" and isinstance(fill, int):
                    dtype = torch.int64
                else:
                    dtype = torch.get_default_dtype()
            return outer._guarded(shape, dtype, torch.device(device), fill, name)

        return like if name.endswith("_like") else sized

    def __enter__(self) -> "CanaryAllocations":
        for name in self._FUNCS:
            self._orig[name] = getattr(torch, name)
        for name in self._FUNCS:
            setattr(torch, name, self._wrap(name))
        return self

    def __exit__(self, *exc):
        for name, fn in self._orig.items():
            setattr(torch, name, fn)
        return False

    # -- verification ----------------------------------------------------------------------------------------------------
    def violations(self) -> List[str]:
        """descriptions of the damaged guards (synchronises the devices involved)"""
        if any(r[0].is_cuda for r in self.records):
            torch.cuda.synchronize()
        bad = []
        for raw, g, payload, what in self.records:
            for side, region, base in (("before", raw[:g], -g), ("after", raw[g + payload:], payload)):
                wrong = (region != PATTERN).nonzero()
                if wrong.numel():
                    first = int(wrong[0]) if side == "after" else int(wrong[-1])
                    bad.append("%s: %i bytes damaged %s the tensor, nearest at byte offset %i" % (what, int(wrong.numel()), side, base + first))
        return bad

    def check(self):
        """raise :class:`GuardViolation` when a guard was written"""
        bad = self.violations()
        if bad:
            raise GuardViolation("out-of-bounds writes:\n  " + "\n  ".join(bad))

    def num_guarded(self) -> int:
        """how many allocations were guarded"""
        return len(self.records)


def _flatten(res) -> List[torch.Tensor]:
    if isinstance(res, torch.Tensor):
        return [res]
    if isinstance(res, (tuple, list)):
        out = []
        for r in res:
            out += _flatten(r)
        return out
    return []


def check_repeatable(fn: Callable[[], Any], *, atol: float = 0.0, rtol: float = 0.0) -> None:
    """``fn()`` twice on the same inputs: equal results (bit-wise with the default tolerances)"""
    a = [t.detach().clone() for t in _flatten(fn())]
    b = _flatten(fn())
    assert len(a) == len(b)
    for i, (x, y) in enumerate(zip(a, b)):
        if atol == 0.0 and rtol == 0.0:
            assert torch.equal(x, y), "result %i differs between two runs on the same inputs (max abs diff %g)" % (i, float((x.float() - y.float()).abs().max()))
        else:
            torch.testing.assert_close(y, x, atol=atol, rtol=rtol)


def check_stream_order(make_inputs: Callable[[], Sequence[torch.Tensor]], fn: Callable[..., Any], *, atol: float = 0.0, rtol: float = 0.0,
                       spin_cycles: int = 20_000_000) -> None:
    """
    ``fn(*inputs)`` on the current stream against the same on a side stream under adverse timing: the inputs are produced by a
    third stream behind a spin kernel, the side stream only depends on them through an event. A kernel that is launched on a
    stream other than the current one, or a wrapper that touches its inputs early, produces a different (stale) result.

    :param make_inputs: returns fresh CUDA input tensors (called twice; must be deterministic)
    """
    ref = [t.detach().clone() for t in _flatten(fn(*make_inputs()))]
    torch.cuda.synchronize()
    producer, side = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(producer):
        torch.cuda._sleep(spin_cycles)
        inputs = [t for t in make_inputs()]
        ready = torch.cuda.Event()
        ready.record(producer)
    with torch.cuda.stream(side):
        side.wait_event(ready)
        for t in inputs:
            t.record_stream(side)
        out = _flatten(fn(*inputs))
        done = torch.cuda.Event()
        done.record(side)
    # consumer on the default stream, again only through an event
    torch.cuda.current_stream().wait_event(done)
    got = [t.detach().clone() for t in out]
    torch.cuda.synchronize()
    assert len(got) == len(ref)
    for i, (x, y) in enumerate(zip(ref, got)):
        if atol == 0.0 and rtol == 0.0:
            assert torch.equal(x, y), "result %i differs under the delayed-stream schedule (max abs diff %g)" % (i, float((x.float() - y.float()).abs().max()))
        else:
            torch.testing.assert_close(y, x, atol=atol, rtol=rtol)
