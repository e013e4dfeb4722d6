"""
Callback interface for ``task = "forward"``.  Parity: returnn/forward_iface.py:15-39.
"""

from __future__ import annotations
from .tensor import TensorDict


class ForwardCallbackIface:
    """``init`` once, ``process_seq`` per sequence (outputs as numpy, padding removed), ``finish`` at the end"""

    def init(self, *, model):
        """before the first sequence"""

    def process_seq(self, *, seq_tag: str, outputs: TensorDict):
        """one sequence"""
        raise NotImplementedError

    def finish(self):
        """after the last sequence"""
