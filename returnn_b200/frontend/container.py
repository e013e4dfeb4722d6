"""
Module containers.  Parity: returnn/frontend/container.py (ModuleList, Sequential, ParameterList, sequential).
"""

from __future__ import annotations
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Union, TypeVar, Generic
from .module import Module, Functional
from .parameter import Parameter

__all__ = ["ModuleList", "Sequential", "ParameterList", "sequential"]

_UnaryFunc = Callable
__ModT = TypeVar("__ModT", bound=Module)


def _convert(item) -> Module:
    if isinstance(item, Module):
        return item
    if callable(item):
        return Functional(item)
    raise TypeError("ModuleList: invalid item %r" % (item,))


class ModuleList(Module):
    """list of modules; items are attributes "0", "1", ... (or the dict keys)"""

    def __init__(self, *modules):
        super().__init__()
        if len(modules) == 1 and isinstance(modules[0], dict):
            for k, v in modules[0].items():
                setattr(self, k, _convert(v))
        elif len(modules) == 1 and isinstance(modules[0], ModuleList):
            for k, v in modules[0]._get_modules().items():
                setattr(self, k, v)
        elif len(modules) == 1 and not isinstance(modules[0], Module) and isinstance(modules[0], Iterable) and not callable(modules[0]):
            for i, m in enumerate(modules[0]):
                setattr(self, str(i), _convert(m))
        else:
            for i, m in enumerate(modules):
                setattr(self, str(i), _convert(m))

    def _get_modules(self) -> Dict[str, Module]:
        return {k: v for k, v in vars(self).items() if isinstance(v, Module)}

    def append(self, module: Module) -> "ModuleList":
        """add at end"""
        setattr(self, str(len(self)), _convert(module))
        return self

    def extend(self, modules: Iterable[Module]) -> "ModuleList":
        """add many"""
        for m in modules:
            self.append(m)
        return self

    def __len__(self) -> int:
        return len(self._get_modules())

    def __iter__(self) -> Iterator[Module]:
        return iter(self._get_modules().values())

    def __delitem__(self, key):
        if isinstance(key, slice):
            for k in list(self._get_modules().keys())[key]:
                delattr(self, k)
        else:
            delattr(self, list(self._get_modules().keys())[key])

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            keys = list(self._get_modules().keys())[idx]
            return self.__class__({k: getattr(self, k) for k in keys})
        if isinstance(idx, str):
            return getattr(self, idx)
        return list(self._get_modules().values())[idx]

    def __setitem__(self, idx, module):
        key = list(self._get_modules().keys())[idx]
        setattr(self, key, _convert(module))

    __call__ = Module.__call__


class Sequential(ModuleList):
    """calls the modules one after the other"""

    def __call__(self, inp, *, collected_outputs: Optional[Dict[str, object]] = None, **kwargs):
        for name, module in self._get_modules().items():
            inp = module(inp, **kwargs)
            if collected_outputs is not None:
                collected_outputs[name] = inp
        return inp


class ParameterList(Module):
    """list of parameters"""

    def __init__(self, *parameters):
        super().__init__()
        if len(parameters) == 1 and isinstance(parameters[0], dict):
            for k, v in parameters[0].items():
                setattr(self, k, v)
        elif len(parameters) == 1 and not isinstance(parameters[0], Parameter) and isinstance(parameters[0], Iterable):
            for i, p in enumerate(parameters[0]):
                setattr(self, str(i), p)
        else:
            for i, p in enumerate(parameters):
                setattr(self, str(i), p)

    def _get_parameters(self) -> Dict[str, Parameter]:
        return {k: v for k, v in vars(self).items() if isinstance(v, Parameter)}

    def append(self, parameter: Parameter) -> "ParameterList":
        """add at end"""
        setattr(self, str(len(self)), parameter)
        return self

    def extend(self, parameters: Iterable[Parameter]) -> "ParameterList":
        """add many"""
        for p in parameters:
            self.append(p)
        return self

    def __len__(self) -> int:
        return len(self._get_parameters())

    def __iter__(self) -> Iterator[Parameter]:
        return iter(self._get_parameters().values())

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            keys = list(self._get_parameters().keys())[idx]
            return self.__class__({k: getattr(self, k) for k in keys})
        return list(self._get_parameters().values())[idx]

    def __setitem__(self, idx, parameter):
        key = list(self._get_parameters().keys())[idx]
        setattr(self, key, parameter)

    __call__ = Module.__call__


def sequential(source, *modules):
    """apply modules (or functions) one after the other"""
    for m in modules:
        source = m(source)
    return source
