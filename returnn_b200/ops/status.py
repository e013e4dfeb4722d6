"""
Status board: where the kernels with bounded waits report that a wait ran out.

Several kernel families give up a wait after a limit instead of spinning forever (the tcgen05 GEMMs and the persistent
LSTM on their mbarriers and grid barriers, the NVLink all-reduce and parameter-averaging kernels on their cross-rank
flags). A kernel that gives up writes a code into a device word and skips its data phase, so its output is not valid.
All those words live in ONE small int32 tensor per device, the board, so that the training loop can copy the whole
board to pinned host memory with a single asynchronous copy per step, next to the deferred loss read, and raise
:class:`KernelWaitTimeout` one step late without any extra synchronisation.

Slots (``SLOT_*``): each family owns one word; ``describe`` turns a code into a message.
"""

from __future__ import annotations
from typing import Callable, Dict, List, Optional, Tuple
import torch

SLOT_GEMM = 0  # tcgen05 GEMM family, attention GEMMs, persistent LSTM, native encoder executor
SLOT_ALLREDUCE = 1  # fused gradient all-reduce
SLOT_PARAM_AVG = 2  # fused AdamW + parameter averaging
SLOT_SMALL_REDUCE = 3  # small-vector all-reduce (batch-norm statistics)
SLOT_USER = 4  # first slot free for other kernels
NUM_SLOTS = 16

_boards: Dict[str, torch.Tensor] = {}
_describers: Dict[int, Callable[[int], str]] = {}


class KernelWaitTimeout(RuntimeError):
    """a kernel gave up a bounded wait: its results (and everything computed from them) are not valid"""

    def __init__(self, msg: str, codes: Optional[Dict[int, int]] = None):
        super().__init__(msg)
        self.codes = dict(codes or {})


def _key(device) -> str:
    d = torch.device(device)
    if d.type == "cuda" and d.index is None:
        d = torch.device("cuda", torch.cuda.current_device())
    return str(d)


def board(device) -> torch.Tensor:
    """the int32 ``[NUM_SLOTS]`` status tensor of ``device`` (created zeroed on first use)"""
    key = _key(device)
    t = _boards.get(key)
    if t is None:
        t = torch.zeros(NUM_SLOTS, dtype=torch.int32, device=device)
        _boards[key] = t
    return t


def word(device, slot: int) -> torch.Tensor:
    """one-element view of the board: pass ``word(...).data_ptr()`` to a kernel as its status pointer"""
    assert 0 <= slot < NUM_SLOTS
    return board(device)[slot: slot + 1]


def register_describer(slot: int, fn: Callable[[int], str]):
    """``fn(code) -> text`` for the messages of :func:`raise_if_set`"""
    _describers[slot] = fn


def _describe_gemm(v: int) -> str:
    return "tcgen05 GEMM / persistent LSTM: bounded wait ran out (role %i, position %i)" % ((v >> 24) & 0xFF, v & 0xFFFFFF)


def _describe_collective(name: str) -> Callable[[int], str]:
    def fn(v: int) -> str:
        return "%s: peer rank %i was not seen at the %s barrier of CTA %i within the wait limit" % (
            name, (v >> 16) & 0xFF, "entry" if ((v >> 24) & 0xFF) == 1 else "exit", v & 0xFFFF)

    return fn


register_describer(SLOT_GEMM, _describe_gemm)
register_describer(SLOT_ALLREDUCE, _describe_collective("fused gradient all-reduce"))
register_describer(SLOT_PARAM_AVG, _describe_collective("fused parameter averaging"))
register_describer(SLOT_SMALL_REDUCE, _describe_collective("small-vector all-reduce"))


def describe(slot: int, code: int) -> str:
    """message for a non-zero code in a slot"""
    fn = _describers.get(slot)
    return fn(code) if fn is not None else "kernel status slot %i: code 0x%x" % (slot, code)


def raise_if_set(values: List[int], *, device=None, where: str = ""):
    """
    :param values: host copy of a board
    :param device: if given, the board of this device is cleared before raising (the error was reported; the next step starts clean)
    """
    bad = {i: int(v) for i, v in enumerate(values) if int(v) != 0}
    if not bad:
        return
    if device is not None:
        board(device).zero_()
    msg = "; ".join(describe(i, v) for i, v in sorted(bad.items()))
    raise KernelWaitTimeout("%s%s. The affected step's results are not valid." % (where + ": " if where else "", msg), bad)


def check_now(device=None):
    """synchronising check of one device's board (or all): for tests, benchmarks and the end of an epoch"""
    for key, t in list(_boards.items()):
        if device is not None and key != _key(device):
            continue
        raise_if_set(t.tolist(), device=key)


class StatusPoller:
    """
    Per-step asynchronous read of a device's board. ``step()``, called after a step's kernels were queued, starts the copy of
    the board into a pinned two-slot ring and then looks at the copy made one step earlier, which has long finished by then:
    a timeout is raised one step late and the host never waits for the device. ``flush()`` checks what is still pending.
    """

    def __init__(self, device):
        self.device = torch.device(device)
        self._ring: List[Tuple[torch.Tensor, "torch.cuda.Event"]] = []
        self._pending: List[int] = []
        self._i = 0

    def step(self, *, where: str = ""):
        """queue the copy of the board as of the current stream position; check the copy of the step before"""
        if self.device.type != "cuda" or _key(self.device) not in _boards:
            return
        if not self._ring:
            self._ring = [(torch.zeros(NUM_SLOTS, dtype=torch.int32).pin_memory(), torch.cuda.Event()) for _ in range(2)]
        host, ev = self._ring[self._i]
        host.copy_(board(self.device), non_blocking=True)
        ev.record()
        self._pending.append(self._i)
        self._i ^= 1
        while len(self._pending) > 1:
            self._check_oldest(where)

    def flush(self, *, where: str = ""):
        """wait for every copy still pending and raise :class:`KernelWaitTimeout` if a kernel reported"""
        while self._pending:
            self._check_oldest(where)

    def _check_oldest(self, where: str):
        i = self._pending.pop(0)
        host, ev = self._ring[i]
        ev.synchronize()
        raise_if_set(host.tolist(), device=self.device, where=where)
