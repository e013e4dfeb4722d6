"""
Graph utilities of the frontend API. Execution here is eager: a tensor records neither its inputs nor its consumers, so the
dependency queries return empty lists (as the reference's eager torch backend does); ``walk_tensor_consumers`` therefore visits
the seeds only.  Reference: returnn/frontend/graph.py.
"""

from __future__ import annotations
from typing import Callable, List, Optional, Sequence, Union
from ..tensor import Tensor

__all__ = ["get_tensor_dependencies", "get_tensor_consumers", "walk_tensor_consumers"]


def get_tensor_dependencies(x: Tensor) -> Sequence[Tensor]:
    """inputs of ``x`` (none are recorded in eager execution)"""
    return []


def get_tensor_consumers(x: Tensor) -> Sequence[Tensor]:
    """tensors computed from ``x`` (none are recorded in eager execution)"""
    return []


def walk_tensor_consumers(seed: Union[Tensor, Sequence[Tensor]], *, filter_outputs: Optional[Callable[[Tensor], bool]] = None,
                          ending_condition: Optional[Callable[[Tensor], bool]] = None) -> List[Tensor]:
    """breadth-first over the consumers of ``seed``"""
    seen = set()
    queue = [seed] if isinstance(seed, Tensor) else list(seed)
    out: List[Tensor] = []
    while queue:
        x = queue.pop(0)
        if id(x) in seen:
            continue
        seen.add(id(x))
        if filter_outputs is None or filter_outputs(x):
            out.append(x)
        if ending_condition is not None and ending_condition(x):
            break
        queue.extend(get_tensor_consumers(x))
    return out
