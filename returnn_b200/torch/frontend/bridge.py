"""
Bridge between ``rf.Module`` and ``torch.nn.Module``: the RF module tree is mirrored as a torch module tree so that
``state_dict()`` keys are the RF attribute paths; auxiliary parameters become buffers.

Parity: returnn/torch/frontend/bridge.py:37-207.
"""

from __future__ import annotations
from typing import Optional
import torch
from ... import frontend as rf
from ...tensor import Tensor, Dim


def pt_module_to_rf_module(pt_module: torch.nn.Module) -> rf.Module:
    """wrap a torch module"""
    if isinstance(pt_module, RFModuleAsPTModule):
        return pt_module.rf_module
    return PTModuleAsRFModule(pt_module=pt_module)


def pt_module_to_wrapped_rf_module(pt_module: torch.nn.Module) -> Optional[rf.Module]:
    """the wrapped RF module if pt_module is a wrapper"""
    if isinstance(pt_module, RFModuleAsPTModule):
        return pt_module.rf_module
    return None


def rf_module_to_pt_module(rf_module: rf.Module, *, aux_params_as_buffers: bool = True) -> torch.nn.Module:
    """wrap an RF module"""
    if isinstance(rf_module, PTModuleAsRFModule):
        return rf_module.pt_module
    return RFModuleAsPTModule(rf_module=rf_module, aux_params_as_buffers=aux_params_as_buffers)


class PTModuleAsRFModule(rf.Module):
    """a torch module inside an RF module tree; its parameters show up as rf.Parameter with anonymous dims"""

    def __init__(self, pt_module: torch.nn.Module):
        super().__init__()
        self._pt_module = pt_module
        for name, p in pt_module.named_parameters(recurse=True):
            dims = [Dim(s, name="%s:dim%i" % (name, i)) for i, s in enumerate(p.shape)]
            rp = rf.Parameter(dims, dtype=str(p.dtype).split(".")[-1], raw_tensor=p, trainable=p.requires_grad)
            setattr(self, name.replace(".", "__"), rp)

    @property
    def pt_module(self) -> torch.nn.Module:
        """the torch module"""
        return self._pt_module

    def __call__(self, *args, **kwargs):
        return self._pt_module(*args, **kwargs)


class RFModuleAsPTModule(torch.nn.Module):
    """the RF module tree mirrored as torch modules"""

    def __init__(self, rf_module: rf.Module, *, aux_params_as_buffers: bool = True):
        super().__init__()
        self._rf_module = rf_module
        self._aux_params_as_buffers = aux_params_as_buffers
        self._is_initializing = True
        for name, rf_param in _direct_params(rf_module):
            raw = rf_param.raw_tensor
            if rf_param.auxiliary and aux_params_as_buffers:
                data = raw.data if isinstance(raw, torch.nn.Parameter) else raw
                self.register_buffer(name, data)
                rf_param._raw_tensor = data
            else:
                if not isinstance(raw, torch.nn.Parameter):
                    raw = torch.nn.Parameter(raw, requires_grad=rf_param.trainable)
                    rf_param._raw_tensor = raw
                self.register_parameter(name, raw)
        for name, rf_mod in rf_module.named_children():
            if name.startswith("_param_"):
                # parametrization holder: expose the raw parameter under its original name
                for pname, p in _direct_params(rf_mod):
                    self.register_parameter(pname, p.raw_tensor)
                continue
            self.add_module(name, rf_module_to_pt_module(rf_mod, aux_params_as_buffers=aux_params_as_buffers))
        self._is_initializing = False

    def _get_name(self):
        return self._rf_module.__class__.__name__ + "[RF→PT]"

    @property
    def rf_module(self) -> rf.Module:
        """the RF module"""
        return self._rf_module

    def forward(self, *args, **kwargs):
        return self._rf_module(*args, **kwargs)

    def _apply(self, fn, *args, **kwargs):
        super()._apply(fn, *args, **kwargs)
        # .to()/.cuda() may replace parameter or buffer objects: keep the RF side pointing at the live tensors
        for name, rf_param in _direct_params(self._rf_module):
            if name in self._parameters and self._parameters[name] is not None:
                rf_param._raw_tensor = self._parameters[name]
            elif name in self._buffers and self._buffers[name] is not None:
                rf_param._raw_tensor = self._buffers[name]
            raw = rf_param._raw_tensor
            rf_param.dtype = str(raw.dtype).split(".")[-1]
        return self

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        for name, rf_param in _direct_params(self._rf_module):
            if name in self._buffers and self._buffers[name] is not None:
                rf_param._raw_tensor = self._buffers[name]


def _direct_params(rf_module: rf.Module):
    for name, value in vars(rf_module).items():
        if isinstance(value, rf.Parameter):
            yield name, value
