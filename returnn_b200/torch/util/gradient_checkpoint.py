"""
``gradient_checkpoint_scope``: tensors created inside the scope are not stored for backward; when backward needs one,
the recorded ops of the scope are replayed (with the RNG state restored) to recompute it.

Implementation: ``torch.autograd.graph.saved_tensors_hooks`` inside the scope replace every saved tensor that was created
in the scope by a handle into a per-scope tape of (function, args) recorded through ``TorchDispatchMode``; unpacking replays
the tape up to the needed tensor once and caches the results until backward has consumed them.

Parity: returnn/torch/util/gradient_checkpoint.py:94 (same semantics; own implementation).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Tuple
import weakref
import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_map


class _Tape:
    def __init__(self):
        self.entries: List[Tuple[Any, tuple, dict, List[int]]] = []  # func, args, kwargs, ids of outputs
        self.produced: Dict[int, Tuple[int, int]] = {}  # tensor id -> (entry idx, output idx)
        self.cache: Optional[Dict[Tuple[int, int], torch.Tensor]] = None
        self.rng_cpu = torch.get_rng_state()
        self.rng_cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None
        self.keep: List[torch.Tensor] = []  # inputs from outside the scope stay alive through args
        self.num_unpacked = 0
        self.num_packed = 0

    def replay(self):
        """recompute everything recorded in the scope"""
        cache: Dict[Tuple[int, int], torch.Tensor] = {}
        live: Dict[int, torch.Tensor] = {}
        cpu_state = torch.get_rng_state()
        cuda_state = torch.cuda.get_rng_state() if self.rng_cuda is not None else None
        torch.set_rng_state(self.rng_cpu)
        if self.rng_cuda is not None:
            torch.cuda.set_rng_state(self.rng_cuda)
        try:
            with torch.no_grad():
                for ei, (func, args, kwargs, out_ids) in enumerate(self.entries):
                    def sub(x):
                        if isinstance(x, _Ref):
                            return live[x.tid]
                        return x

                    out = func(*tree_map(sub, args), **tree_map(sub, kwargs))
                    outs = out if isinstance(out, (tuple, list)) else [out]
                    for oi, (o, tid) in enumerate(zip(outs, out_ids)):
                        if isinstance(o, torch.Tensor):
                            live[tid] = o
                            cache[(ei, oi)] = o
        finally:
            torch.set_rng_state(cpu_state)
            if cuda_state is not None:
                torch.cuda.set_rng_state(cuda_state)
        self.cache = cache


class _Ref:
    """placeholder in the tape for a tensor produced earlier in the same scope"""

    __slots__ = ("tid",)

    def __init__(self, tid: int):
        self.tid = tid


class _Record(TorchDispatchMode):
    def __init__(self, tape: _Tape):
        super().__init__()
        self.tape = tape

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        tape = self.tape

        def ref(x):
            if isinstance(x, torch.Tensor) and id(x) in tape.produced:
                return _Ref(id(x))
            return x

        outs = out if isinstance(out, (tuple, list)) else [out]
        out_ids = [id(o) for o in outs]
        ei = len(tape.entries)
        tape.entries.append((func, tree_map(ref, args), tree_map(ref, kwargs), out_ids))
        for oi, o in enumerate(outs):
            if isinstance(o, torch.Tensor):
                tape.produced[id(o)] = (ei, oi)
                tape.keep.append(o)  # ids must stay unique while recording
        return out


class gradient_checkpoint_scope:
    """context manager, see module docstring"""

    def __init__(self):
        self.tape = _Tape()
        self._record = _Record(self.tape)
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
        self._active = False

    def _pack(self, x: torch.Tensor):
        tape = self.tape
        key = tape.produced.get(id(x)) if self._active or True else None
        if key is not None and x.requires_grad is False or (key is not None):
            tape.num_packed += 1
            return ("tape", key, x.shape, x.dtype)
        return ("raw", x)

    def _unpack(self, packed):
        if packed[0] == "raw":
            return packed[1]
        _, key, _, _ = packed
        tape = self.tape
        if tape.cache is None:
            tape.replay()
        out = tape.cache[key]
        tape.num_unpacked += 1
        if tape.num_unpacked >= tape.num_packed:
            tape.cache = None
            tape.num_unpacked = 0
        return out

    def __enter__(self):
        self._active = True
        self._hooks.__enter__()
        self._record.__enter__()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self._record.__exit__(exc_type, exc_val, exc_tb)
        # keep the saved-tensor hooks active for ops that consume scope tensors right after the scope:
        # they are registered per saved tensor at save time, so exiting here is enough for later ops
        self._hooks.__exit__(exc_type, exc_val, exc_tb)
        self._active = False
        # drop strong refs to the intermediates: this is the memory saving
        self.tape.keep.clear()
        return False
