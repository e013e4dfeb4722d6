"""
Helpers for interactive debugging: find live objects of a class on the Python stacks; a tiny HDF writer for dumps.

Parity: returnn/util/debug_helpers.py (find_obj_in_stack :11, SimpleHdf :53).
"""

from __future__ import annotations
from typing import Optional, Union
import sys
import types


def find_obj_in_stack(cls, stack: Optional[Union[types.FrameType, types.TracebackType]] = None, all_threads: bool = True):
    """:return: the first local variable that is an instance of ``cls``, searching the given stack (or all threads' stacks)"""
    if stack is None and all_threads:
        for frame in sys._current_frames().values():
            obj = find_obj_in_stack(cls, stack=frame)
            if obj is not None:
                return obj
        return None
    if stack is None:
        stack = sys._getframe(1)
    frames = []
    if isinstance(stack, types.TracebackType):
        tb = stack
        while tb is not None:
            frames.append(tb.tb_frame)
            tb = tb.tb_next
    else:
        f = stack
        while f is not None:
            frames.append(f)
            f = f.f_back
    for f in frames:
        for v in f.f_locals.values():
            if isinstance(v, cls):
                return v
    return None


class SimpleHdf:
    """``update({name: array})`` appends datasets to one HDF file (needs h5py)"""

    def __init__(self, filename: str):
        import h5py

        self.hdf = h5py.File(filename, "w")
        self.seq_tag_to_idx = {}
        self.num_seqs = 0

    def update(self, seq_tag: str, data: dict):
        """one group per sequence"""
        if seq_tag not in self.seq_tag_to_idx:
            self.seq_tag_to_idx[seq_tag] = self.num_seqs
            self.num_seqs += 1
        grp = self.hdf.require_group("seq-%i" % self.seq_tag_to_idx[seq_tag])
        grp.attrs["seq_tag"] = seq_tag
        for k, v in data.items():
            if k in grp:
                del grp[k]
            grp.create_dataset(k, data=v)

    def close(self):
        self.hdf.close()
