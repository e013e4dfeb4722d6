"""
Backend selection API kept for config compatibility: there is exactly one backend, torch.
Parity: returnn/frontend/_backend.py:1883-1962 (select_backend_*).
"""

from __future__ import annotations


def select_backend_torch():
    """no-op: torch is the only backend"""
    return None


def select_backend_returnn_layers_tf():
    """not available"""
    raise NotImplementedError("this framework has a single backend (torch); TF net-dict layers are not built")


def is_executing_eagerly() -> bool:
    """always eager"""
    return True


def get_backend_name() -> str:
    """'torch'"""
    return "torch"
