"""
Fused gradient all-reduce for one node over NVLink (``csrc/allreduce.cu``): the gradient arena lives in symmetric memory
(every rank can address every rank's copy), and one kernel per bucket sums the ranks' slices through peer pointers or the
NVSwitch multicast mapping (``multimem.ld_reduce`` / ``multimem.st``), scales by ``1/world``, writes the result to all
ranks and accumulates the squared global gradient norm, so neither a scale pass, nor NCCL, nor a norm pass is needed.

``try_create`` returns None when the prerequisites are missing (no CUDA, other ranks on other nodes, symmetric memory not
available, library missing) unless ``required``. Environment: ``RETURNN_B200_ALLREDUCE_MULTIMEM=0`` keeps the kernel
on plain peer loads and stores (tests that let a rank leave use this, together with ``NCCL_NVLS_ENABLE=0``).
"""

from __future__ import annotations
from typing import Optional
import ctypes
import os
import torch
import torch.distributed as dist
from ..ops import _lib
from ..ops import status as _status_board
from .arena import ParamArena

_vp, _i32, _i64, _f32, _u32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint

DEFAULT_WAIT_MS = 20000


def set_wait_ms(ms: Optional[int] = None):
    """
    Time limit of the cross-rank barrier waits inside the NVLink kernels, for launches made from now on. A peer that has not
    arrived within the limit makes the waiting kernel give up: it writes the status word and skips its data phase, and the
    training loop raises ``KernelWaitTimeout`` when it reads the word. Default: ``RETURNN_B200_COLLECTIVE_WAIT_MS`` or 20 s
    (config: ``torch_distributed["fused_wait_ms"]``).
    """
    if ms is None:
        ms = int(os.environ.get("RETURNN_B200_COLLECTIVE_WAIT_MS", DEFAULT_WAIT_MS))
    fn = _lib.bind("rb200_collective_set_wait_ms", [_i32])
    _lib.check(fn(int(ms)), "collective_set_wait_ms")



class FusedAllReduce:
    """bucket reductions on the arena's gradient buffer"""

    def __init__(self, arena: ParamArena, *, rank: int, world: int, group=None, blocks: int = 128, wait_ms: Optional[int] = None):
        import torch.distributed._symmetric_memory as symm_mem

        assert arena.grad_dtype == torch.float32
        self.arena = arena
        self.rank, self.world = rank, world
        # CTAs of a bucket reduction: it shares the SMs with the backward pass it overlaps (RETURNN_B200_ALLREDUCE_BLOCKS overrides)
        self.blocks = int(os.environ.get("RETURNN_B200_ALLREDUCE_BLOCKS", blocks))
        dev = arena.device
        group = group or dist.group.WORLD
        n = (arena.total + 3) // 4 * 4
        self._grad = symm_mem.empty(n, dtype=torch.float32, device=dev)
        self._grad.zero_()
        self._hdl = symm_mem.rendezvous(self._grad, group)
        lib = _lib.get_lib(required=True)
        lib.rb200_fused_allreduce_flag_words.restype = ctypes.c_int
        words = int(lib.rb200_fused_allreduce_flag_words())
        self._flags = symm_mem.empty(words, dtype=torch.int32, device=dev)
        self._flags.zero_()
        self._hdl_flags = symm_mem.rendezvous(self._flags, group)
        self._norm = symm_mem.empty(8, dtype=torch.float32, device=dev)
        self._norm.zero_()
        self._hdl_norm = symm_mem.rendezvous(self._norm, group)
        arena.replace_grad_buffer(self._grad)
        self._bufs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl.buffer_ptrs])
        self._flag_ptrs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl_flags.buffer_ptrs])
        self._norm_ptrs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl_norm.buffer_ptrs])
        # measured on 2 GPUs: plain peer loads / stores 0.75 ms vs 1.11 ms through the multicast mapping for 400 MB; the switch
        # reduction only pays off when more ranks contribute
        default_mc = "1" if world > 2 else "0"
        use_mc = os.environ.get("RETURNN_B200_ALLREDUCE_MULTIMEM", default_mc) == "1"
        mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0) if use_mc else 0
        self.multicast_ptr = mc
        self._epoch = 1
        self._slot = 0
        # Every rank's accumulator receives the same partial sums, but through atomics whose order differs from rank to rank, so the
        # last bits of the ranks' totals differ. The norm that scales the update must be bitwise the same everywhere (or the ranks'
        # parameters drift apart by rounding noise): all ranks read rank 0's accumulator.
        try:
            self._norm_rank0 = self._hdl_norm.get_buffer(0, (8,), torch.float32)
        except Exception:
            self._norm_rank0 = None
        self._status = _status_board.word(dev, _status_board.SLOT_ALLREDUCE)
        self._fn = _lib.bind("rb200_fused_allreduce", [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _i64, _f32, _u32, _i32, _i32, _vp, _vp])
        self.skip_launches = 0  # failure-detection tests: this many following launches are left out (the peers' waits then run out)
        set_wait_ms(wait_ms)
        # all ranks have zeroed their flags and accumulators before anyone's first kernel signals
        torch.cuda.synchronize(dev)
        dist.barrier(group)

    @property
    def mode(self) -> str:
        """``"fused-multimem"`` (reduction inside the NVSwitch) or ``"fused-peer"`` (peer loads and stores)"""
        return "fused-multimem" if self.multicast_ptr else "fused-peer"

    def reduce_bucket(self, b: int, lo: int, hi: int):
        """average ``flat_grad[lo:hi]`` over the ranks, on the current stream; all ranks must call this in the same order"""
        if self.skip_launches > 0:
            self.skip_launches -= 1
            self._epoch += 2
            return
        _lib.check(self._fn(ctypes.addressof(self._bufs), ctypes.addressof(self._flag_ptrs), ctypes.addressof(self._norm_ptrs),
                            self.multicast_ptr or None, self.world, self.rank, lo, hi - lo, 1.0 / self.world, self._epoch, self._slot,
                            self.blocks, self._status.data_ptr(), _lib.stream_ptr()), "fused_allreduce")
        _lib.count_launch()
        self._epoch += 2

    def finish(self) -> torch.Tensor:
        """
        After the last bucket of a step (on the stream that ran them or one that waits for it): the squared global norm of
        the averaged gradient as a device scalar. The accumulator alternates between two slots; the one for the next step
        is cleared here, which is safe because no peer adds to it before its next step's entry barrier with this rank.
        """
        # complete on every rank once the last bucket's kernel has passed its exit barrier (the kernels ahead of this read in stream order)
        src = self._norm_rank0 if self._norm_rank0 is not None else self._norm
        norm_sq = src[self._slot].clone()
        self._slot ^= 1
        self._norm[self._slot].zero_()
        return norm_sq

    def check_status(self):
        """raise ``KernelWaitTimeout`` if a barrier of an earlier call timed out (synchronises; the training loop reads the
        same word asynchronously once per step through the status board)"""
        v = int(self._status.item())
        if v:
            self._status.zero_()
            raise _status_board.KernelWaitTimeout("rank %i: %s" % (self.rank, _status_board.describe(_status_board.SLOT_ALLREDUCE, v)),
                                                  {_status_board.SLOT_ALLREDUCE: v})


class FusedParamAverager:
    """
    Parameter averaging (``reduce_type="param"``) over NVLink, optionally fused with the AdamW update of the sync step:
    one kernel updates this rank's parameters, waits for all ranks and writes the average to everyone.
    The parameter arena moves into symmetric memory.
    """

    def __init__(self, arena: ParamArena, *, rank: int, world: int, group=None, blocks: int = 128, wait_ms: Optional[int] = None):
        import torch.distributed._symmetric_memory as symm_mem

        assert arena.dtype == torch.float32
        self.arena, self.rank, self.world, self.blocks = arena, rank, world, blocks
        dev = arena.device
        group = group or dist.group.WORLD
        n = (arena.total + 3) // 4 * 4
        self._param = symm_mem.empty(n, dtype=torch.float32, device=dev)
        self._param.zero_()
        self._hdl = symm_mem.rendezvous(self._param, group)
        lib = _lib.get_lib(required=True)
        lib.rb200_fused_allreduce_flag_words.restype = ctypes.c_int
        self._flags = symm_mem.empty(int(lib.rb200_fused_allreduce_flag_words()), dtype=torch.int32, device=dev)
        self._flags.zero_()
        self._hdl_flags = symm_mem.rendezvous(self._flags, group)
        self._norm = symm_mem.empty(8, dtype=torch.float32, device=dev)
        self._norm.zero_()
        self._hdl_norm = symm_mem.rendezvous(self._norm, group)
        arena.replace_param_buffer(self._param)
        self._bufs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl.buffer_ptrs])
        self._flag_ptrs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl_flags.buffer_ptrs])
        self._norm_ptrs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl_norm.buffer_ptrs])
        default_mc = "1" if world > 2 else "0"
        use_mc = os.environ.get("RETURNN_B200_ALLREDUCE_MULTIMEM", default_mc) == "1"
        self.multicast_ptr = int(getattr(self._hdl, "multicast_ptr", 0) or 0) if use_mc else 0
        self._epoch = 1
        self._status = _status_board.word(dev, _status_board.SLOT_PARAM_AVG)
        self.pending = False  # set by the distributed context on sync steps; the optimizer then fuses its update with the average
        _u8p = ctypes.c_void_p
        self._fn = _lib.bind("rb200_fused_adamw_param_avg", [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _u32, _i32, _vp, _vp, _vp, _vp, _u8p, _i32,
                                                              _f32, _f32, _f32, _f32, _f32, _f32, _f32, _i32, _f32, _vp, _i32, _vp])
        set_wait_ms(wait_ms)
        torch.cuda.synchronize(dev)
        dist.barrier(group)

    def average(self, adam: Optional[dict] = None):
        """
        Average the parameters over all ranks on the current stream. ``adam``: arguments of the fused AdamW kernel
        (``g, m, v, wd_flags, lr, b1, b2, eps, wd, bc1, bc2, decoupled, clip, norm``) to run the update in the same launch.
        """
        a = adam or {}
        g = a.get("g")
        norm = a.get("norm")
        _lib.check(self._fn(ctypes.addressof(self._bufs), ctypes.addressof(self._flag_ptrs), ctypes.addressof(self._norm_ptrs),
                            self.multicast_ptr or None, self.world, self.rank, self.arena.total, self._epoch, self.blocks, self._status.data_ptr(),
                            g.data_ptr() if g is not None else None, a["m"].data_ptr() if adam else None, a["v"].data_ptr() if adam else None,
                            a["wd_flags"].data_ptr() if adam else None, 1 if (g is not None and g.dtype == torch.bfloat16) else 0,
                            float(a.get("lr", 0.0)), float(a.get("b1", 0.0)), float(a.get("b2", 0.0)), float(a.get("eps", 0.0)), float(a.get("wd", 0.0)),
                            float(a.get("bc1", 1.0)), float(a.get("bc2", 1.0)), 1 if a.get("decoupled", True) else 0, float(a.get("clip", 0.0)),
                            norm.data_ptr() if norm is not None else None, 1 if adam else 0, _lib.stream_ptr()), "fused_adamw_param_avg")
        _lib.count_launch()
        self._epoch += 2
        self.pending = False
        self.arena.invalidate_shadow()

    @property
    def mode(self) -> str:
        """``"fused-multimem"`` or ``"fused-peer"``"""
        return "fused-multimem" if self.multicast_ptr else "fused-peer"

    def check_status(self):
        """raise ``KernelWaitTimeout`` if a barrier timed out (synchronises)"""
        v = int(self._status.item())
        if v:
            self._status.zero_()
            raise _status_board.KernelWaitTimeout("rank %i: %s" % (self.rank, _status_board.describe(_status_board.SLOT_PARAM_AVG, v)),
                                                  {_status_board.SLOT_PARAM_AVG: v})


def try_create_param_averager(arena: ParamArena, *, rank: int, world: int, required: bool = False, group=None,
                              wait_ms: Optional[int] = None) -> Optional[FusedParamAverager]:
    """the fused averager, or None if it cannot be used here"""
    try:
        if arena.device.type != "cuda" or arena.dtype != torch.float32:
            raise RuntimeError("needs a CUDA arena with fp32 parameters")
        lib = _lib.get_lib()
        if lib is None or not hasattr(lib, "rb200_fused_adamw_param_avg"):
            raise RuntimeError("kernel library without the entry point")
        if os.environ.get("RETURNN_B200_FUSED_ALLREDUCE", "1") != "1":
            raise RuntimeError("disabled by RETURNN_B200_FUSED_ALLREDUCE")
        return FusedParamAverager(arena, rank=rank, world=world, group=group, wait_ms=wait_ms)
    except Exception as exc:
        if required:
            raise
        from ..log import log

        print("Fused parameter averaging not available (%s: %s), using torch.distributed." % (type(exc).__name__, exc), file=log.v3)
        return None


class SmallVectorAllReduce:
    """
    Sum of a small fp32 vector over the ranks through symmetric memory (one CTA per rank: flags, peer loads, peer stores):
    the cross-rank exchange of batch-norm statistics (``[C]`` sums, ``[C]`` sums of squares, a count). Latency of one kernel
    instead of a library collective; the same kernel as the gradient all-reduce on a buffer of its own.
    """

    def __init__(self, *, device, rank: int, world: int, capacity: int = 8192, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world, self.capacity = rank, world, capacity
        group = group or dist.group.WORLD
        self._buf = symm_mem.empty(capacity, dtype=torch.float32, device=device)
        self._buf.zero_()
        self._hdl = symm_mem.rendezvous(self._buf, group)
        lib = _lib.get_lib(required=True)
        lib.rb200_fused_allreduce_flag_words.restype = ctypes.c_int
        words = int(lib.rb200_fused_allreduce_flag_words())
        self._flags = symm_mem.empty(words, dtype=torch.int32, device=device)
        self._flags.zero_()
        self._hdl_flags = symm_mem.rendezvous(self._flags, group)
        self._norm = symm_mem.empty(8, dtype=torch.float32, device=device)
        self._norm.zero_()
        self._hdl_norm = symm_mem.rendezvous(self._norm, group)
        self._bufs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl.buffer_ptrs])
        self._flag_ptrs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl_flags.buffer_ptrs])
        self._norm_ptrs = (ctypes.c_longlong * world)(*[int(p) for p in self._hdl_norm.buffer_ptrs])
        self._epoch = 1
        self._status = _status_board.word(device, _status_board.SLOT_SMALL_REDUCE)
        self._fn = _lib.bind("rb200_fused_allreduce", [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _i64, _f32, _u32, _i32, _i32, _vp, _vp])
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def supports(self, x: torch.Tensor) -> bool:
        """fp32 CUDA tensor that fits"""
        return x.is_cuda and x.dtype == torch.float32 and 0 < x.numel() <= self.capacity

    def all_reduce_sum(self, x: torch.Tensor) -> torch.Tensor:
        """:return: new tensor = sum of x over all ranks; every rank must call this in the same order"""
        n = x.numel()
        n4 = (n + 3) // 4 * 4
        self._buf[:n].copy_(x.reshape(-1))
        if n4 > n:
            self._buf[n:n4].zero_()
        # plain peer loads: a few hundred bytes gain nothing from the multicast mapping
        _lib.check(self._fn(ctypes.addressof(self._bufs), ctypes.addressof(self._flag_ptrs), ctypes.addressof(self._norm_ptrs), None, self.world,
                            self.rank, 0, n4, 1.0, self._epoch, 0, 1, self._status.data_ptr(), _lib.stream_ptr()), "small_vector_allreduce")
        _lib.count_launch()
        self._epoch += 2
        return self._buf[:n].clone().reshape(x.shape)


_small_reducer: Optional[SmallVectorAllReduce] = None


def get_small_reducer() -> Optional[SmallVectorAllReduce]:
    """the process-wide small-vector reducer, if :func:`try_create_small_reducer` made one"""
    return _small_reducer


def try_create_small_reducer(*, device, rank: int, world: int, group=None) -> Optional[SmallVectorAllReduce]:
    """create the process-wide reducer for statistics; None (and NCCL is used) where symmetric memory is not available"""
    global _small_reducer
    try:
        lib = _lib.get_lib()
        if torch.device(device).type != "cuda" or lib is None or not hasattr(lib, "rb200_fused_allreduce"):
            raise RuntimeError("needs CUDA and the kernel library")
        if os.environ.get("RETURNN_B200_FUSED_ALLREDUCE", "1") != "1":
            raise RuntimeError("disabled by RETURNN_B200_FUSED_ALLREDUCE")
        _small_reducer = SmallVectorAllReduce(device=device, rank=rank, world=world, group=group)
    except Exception as exc:
        from ..log import log

        print("Small-vector NVLink all-reduce not available (%s: %s), using torch.distributed." % (type(exc).__name__, exc), file=log.v4)
        _small_reducer = None
    return _small_reducer


def try_create(arena: ParamArena, *, rank: int, world: int, required: bool = False, group=None,
               wait_ms: Optional[int] = None) -> Optional[FusedAllReduce]:
    """the fused reducer, or None if it cannot be used here"""
    try:
        if arena.device.type != "cuda" or arena.grad_dtype != torch.float32:
            raise RuntimeError("needs a CUDA arena with fp32 gradients")
        lib = _lib.get_lib()
        if lib is None or not hasattr(lib, "rb200_fused_allreduce"):
            raise RuntimeError("kernel library without the all-reduce entry point")
        if os.environ.get("RETURNN_B200_FUSED_ALLREDUCE", "1") != "1":
            raise RuntimeError("disabled by RETURNN_B200_FUSED_ALLREDUCE")
        return FusedAllReduce(arena, rank=rank, world=world, group=group, wait_ms=wait_ms)
    except Exception as exc:
        if required:
            raise
        from ..log import log

        print("Fused NVLink all-reduce not available (%s: %s), using torch.distributed." % (type(exc).__name__, exc), file=log.v3)
        return None
