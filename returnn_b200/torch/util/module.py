"""
``torch.nn.Module`` surgery.

Parity: returnn/torch/util/module.py (convert_parameters_to_buffers :10, convert_parameter_to_buffer :24).
"""

from __future__ import annotations
from typing import Collection
import torch


def convert_parameter_to_buffer(module: torch.nn.Module, parameter_name: str, *, deep: bool = True, persistent: bool):
    """replace the parameter ``a.b.c`` by a buffer of the same name and value (no gradient, optionally not in the state dict)"""
    if deep and "." in parameter_name:
        head, _, tail = parameter_name.rpartition(".")
        module = module.get_submodule(head)
        parameter_name = tail
    value = getattr(module, parameter_name)
    assert isinstance(value, torch.nn.Parameter), "%r is not a parameter" % parameter_name
    delattr(module, parameter_name)
    module.register_buffer(parameter_name, value.detach(), persistent=persistent)


def convert_parameters_to_buffers(module: torch.nn.Module, parameter_names: Collection[str], *, deep: bool = True, persistent: bool):
    """see :func:`convert_parameter_to_buffer`"""
    for name in parameter_names:
        convert_parameter_to_buffer(module, name, deep=deep, persistent=persistent)
