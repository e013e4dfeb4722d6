"""
Updater: builds the optimizer from the config ``optimizer`` dict and performs the update step.

- ``optimizer = {"class": "adamw", "weight_decay": ..., ...}``: any ``torch.optim`` class by (lower-case) name, a class
  object, a dotted path, or a callable ``(params, **opts)``. On B200, ``adam``/``adamw`` over a flat arena run as one fused
  kernel (``"fused_arena": False`` disables).
- Weight decay param groups: decay only for parameters with ``weight_decay != 0`` on the RF parameter, not in
  ``weight_decay_modules_blacklist`` (default: LayerNorm, Embedding, BatchNorm) and not biases; a custom
  ``weight_decay_custom_include_check(module=, full_param_name=)`` overrides.
- ``learning_rate_multiplier`` per param group via ``optimizer["learning_rate_multiplier"]`` function
  ``(full_param_name=..., **kwargs) -> float``.
- ``dynamic_learning_rate(network=None, global_train_step=, epoch=, epoch_continuous=, learning_rate=, **kwargs)``.
- ``gradient_noise``, ``gradient_clip`` (value), ``gradient_clip_global_norm``, ``log_grad_norm``,
  ``num_allowed_consec_invalid_gradient_steps``, GradScaler.
- Optimizer checkpoint: ``{"optimizer": state_dict, "optimizer_class_name", "optimizer_opts", "param_names", "epoch",
  "step", ...}``; on load, states are re-mapped by parameter name; the old bare ``state_dict`` format is accepted.

Parity: returnn/torch/updater.py (Updater :93, step :257-320, _create_optimizer :478-532,
_get_optimizer_param_groups :544-663, save_optimizer :434-469, load_optimizer :332-422, gradient_noise_ :687-696).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Iterable, List, Optional, Set, Tuple, Type, Union
import gc
import os
import typing
import torch
from ..log import log
from ..utils.basic import get_fwd_compat_kwargs
from .. import frontend as rf

_OptimizerClassesDictInitialized = False
_OptimizerClassesDict: Dict[str, Type[torch.optim.Optimizer]] = {}


def _init_optimizer_classes_dict():
    global _OptimizerClassesDictInitialized
    if _OptimizerClassesDictInitialized:
        return
    _OptimizerClassesDictInitialized = True
    for name, cls in list(vars(torch.optim).items()):
        if isinstance(cls, type) and issubclass(cls, torch.optim.Optimizer) and cls is not torch.optim.Optimizer:
            _OptimizerClassesDict[name.lower()] = cls
    from .optim.lion import Lion

    _OptimizerClassesDict["lion"] = Lion
    from .optim.fused_adamw import FusedArenaAdamW

    _OptimizerClassesDict["fusedarenaadamw"] = FusedArenaAdamW


def get_optimizer_class(class_name) -> Type[torch.optim.Optimizer]:
    """
    :param class_name: name (case-insensitive, "optimizer" suffix optional), dotted path, class, or callable returning a class
    """
    _init_optimizer_classes_dict()
    if isinstance(class_name, type):
        assert issubclass(class_name, torch.optim.Optimizer)
        return class_name
    if callable(class_name):
        return class_name
    assert isinstance(class_name, str)
    if "." in class_name:
        import importlib

        mod_name, _, cls_name = class_name.rpartition(".")
        if mod_name.startswith("returnn."):
            mod_name = "returnn_b200." + mod_name[len("returnn."):]
        return getattr(importlib.import_module(mod_name), cls_name)
    key = class_name.lower()
    if key not in _OptimizerClassesDict and key.endswith("optimizer"):
        key = key[: -len("optimizer")]
    if key not in _OptimizerClassesDict:
        raise ValueError("Optimizer %r not found; have %s" % (class_name, sorted(_OptimizerClassesDict)))
    return _OptimizerClassesDict[key]


def _get_class_init_kwargs(optim_class) -> List[str]:
    import inspect

    names: List[str] = []
    for cls in getattr(optim_class, "__mro__", [optim_class]):
        init = getattr(cls, "__init__", None)
        if init is None:
            continue
        try:
            for n, p in inspect.signature(init).parameters.items():
                if n not in ("self", "params") and p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY) and n not in names:
                    names.append(n)
        except (TypeError, ValueError):
            pass
    return names


class Updater:
    """owns the optimizer; ``step()`` applies one update"""

    def __init__(self, *, config, network: torch.nn.Module, device: torch.device, initial_learning_rate: float = 1.0):
        self.config = config
        self.learning_rate = float(initial_learning_rate)
        self._effective_learning_rate = self.learning_rate
        self.network = network
        self._device = device
        self._current_train_step = 0
        self._current_epoch = 1
        self._current_epoch_continuous = 0.0
        self.learning_rate_function: Optional[Callable] = self.config.typed_value("dynamic_learning_rate", None)
        if self.learning_rate_function is not None:
            print("Using dynamic learning rate scheduler that updates based on global train steps", file=log.v2)
            if not callable(self.learning_rate_function):
                raise NotImplementedError("dynamic_learning_rate must be callable, got %r" % type(self.learning_rate_function))
        self._optimizer_opts = None
        self.optimizer: Optional[torch.optim.Optimizer] = None
        self._grad_clip = self.config.float("gradient_clip", 0.0)
        self._grad_clip_global_norm = self.config.float("gradient_clip_global_norm", 0.0)
        self._grad_noise = self.config.float("gradient_noise", 0.0)
        self._grad_noise_generator: Optional[torch.Generator] = None
        self._num_allowed_consec_invalid_gradient_steps = self.config.typed_value("num_allowed_consec_invalid_gradient_steps", None)
        self._num_consec_invalid_gradient_steps = 0
        self._log_grad_norm = self.config.bool("log_grad_norm", False)
        self._last_grad_norm: Optional[torch.Tensor] = None
        self._arena = None
        self._precomputed_grad_norm_sq: Optional[torch.Tensor] = None

    def set_learning_rate(self, value: float):
        """base learning rate of the epoch"""
        self.learning_rate = float(value)
        self._update_effective_learning_rate()

    def get_effective_learning_rate(self) -> float:
        """after dynamic_learning_rate"""
        return self._effective_learning_rate

    def _update_effective_learning_rate(self):
        self._effective_learning_rate = self.learning_rate
        if self.learning_rate_function is not None:
            self._effective_learning_rate = float(self.learning_rate_function(
                network=None, global_train_step=self._current_train_step, epoch=self._current_epoch,
                epoch_continuous=self._current_epoch_continuous, learning_rate=self.learning_rate, **get_fwd_compat_kwargs()))
        if self.optimizer:
            for group in self.optimizer.param_groups:
                group["lr"] = self._effective_learning_rate * group.get("learning_rate_multiplier", 1.0)

    def set_current_train_step(self, *, global_train_step: int, epoch: int, epoch_continuous: Optional[float] = None):
        """called every step; updates the dynamic learning rate"""
        self._current_train_step = global_train_step
        self._current_epoch = epoch
        self._current_epoch_continuous = epoch_continuous
        self._update_effective_learning_rate()

    def set_arena(self, arena):
        """flat arena of the distributed context (so that optimizer and reducer share one)"""
        self._arena = arena

    def zero_grad(self):
        """
        Clear the gradients before a step. While a flat arena is active (distributed reduction or the arena optimizer), the
        gradients must stay views of the arena for EVERY optimizer class: the bucket reductions work on arena slices, so a
        ``zero_grad(set_to_none=True)`` of a torch optimizer, after which autograd allocates fresh gradient tensors, would
        detach them from what is being reduced. One memset of the arena, then every ``param.grad`` is re-pointed to its view.
        """
        arena = self._arena if self._arena is not None else getattr(self.optimizer, "arena", None)
        if arena is not None:
            arena.zero_grad()
            arena.relink_grads()
            return
        self.optimizer.zero_grad()

    def set_precomputed_grad_norm_sq(self, value: Optional[torch.Tensor]):
        """squared global grad norm delivered by the fused gradient reduction (saves the extra pass)"""
        self._precomputed_grad_norm_sq = value

    def step(self, *, grad_scaler: Optional[torch.amp.GradScaler] = None) -> Optional[torch.Tensor]:
        """
        unscale, noise, clip, check for inf/nan, optimizer step.
        :return: global grad norm (device scalar) if it was computed
        """
        if grad_scaler is not None:
            grad_scaler.unscale_(self.optimizer)
        fused_opt = getattr(self.optimizer, "is_fused_arena", False)
        if fused_opt and not self._grad_noise and not self._grad_clip:
            params = None  # the arena optimizer works on the flat buffers: no per-parameter list needed in the step
        else:
            params = [p for p in self.network.parameters() if p.grad is not None]
        if self._grad_noise:
            gradient_noise_(params, self._grad_noise, generator=self._get_noise_generator())
        if self._grad_clip:
            torch.nn.utils.clip_grad_value_(params, self._grad_clip)
        grad_norm = None
        need_norm = self._grad_clip_global_norm or self._log_grad_norm or self._num_allowed_consec_invalid_gradient_steps is not None
        if need_norm:
            if self._precomputed_grad_norm_sq is not None:
                grad_norm = torch.sqrt(self._precomputed_grad_norm_sq)
            elif fused_opt:
                grad_norm = self.optimizer.grad_norm()
            else:
                grad_norm = torch.nn.utils.get_total_norm([p.grad for p in params], norm_type=2.0) if hasattr(torch.nn.utils, "get_total_norm") else _total_norm(params)
        self._precomputed_grad_norm_sq = None
        if self._grad_clip_global_norm:
            if fused_opt:
                self.optimizer.set_clip(self._grad_clip_global_norm, grad_norm)
            else:
                coef = torch.clamp(self._grad_clip_global_norm / (grad_norm + 1e-6), max=1.0)
                torch._foreach_mul_([p.grad for p in params], coef.to(params[0].grad.dtype))
        self._last_grad_norm = grad_norm
        if self._num_allowed_consec_invalid_gradient_steps is not None and grad_norm is not None:
            if not bool(torch.isfinite(grad_norm)):
                self._num_consec_invalid_gradient_steps += 1
                print("Invalid gradient norm %s in step %i (%i consecutive), skipping the update" % (
                    float(grad_norm), self._current_train_step, self._num_consec_invalid_gradient_steps), file=log.v2)
                if self._num_consec_invalid_gradient_steps > self._num_allowed_consec_invalid_gradient_steps:
                    raise RuntimeError("Got %i invalid gradients in succession, abort training" % self._num_consec_invalid_gradient_steps)
                self.zero_grad()
                return grad_norm
            self._num_consec_invalid_gradient_steps = 0
        if grad_scaler is not None:
            grad_scaler.step(self.optimizer)
            grad_scaler.update()
        else:
            self.optimizer.step()
        return grad_norm

    def get_last_grad_norm(self) -> Optional[torch.Tensor]:
        """grad norm of the last step (device scalar)"""
        return self._last_grad_norm

    def _get_noise_generator(self) -> torch.Generator:
        if self._grad_noise_generator is None:
            self._grad_noise_generator = torch.Generator(device=self._device)
            self._grad_noise_generator.manual_seed(self.config.int("random_seed", 42) + 7919)
        return self._grad_noise_generator

    def create_optimizer(self):
        """from config ``optimizer``"""
        optimizer_opts = self.config.typed_value("optimizer", None)
        if optimizer_opts is None:
            raise ValueError("config field 'optimizer' needs to be set explicitly for the torch engine")
        self._optimizer_opts = optimizer_opts
        self.optimizer = self._create_optimizer(optimizer_opts)
        self._update_effective_learning_rate()

    def load_optimizer(self, filename: str):
        """load the optimizer state, re-mapping by parameter names when the file has them"""
        print("Load optimizer %s" % filename, file=log.v4)
        ckpt = torch.load(filename, map_location=self._device, weights_only=False)
        if isinstance(ckpt, dict) and "optimizer" in ckpt and "param_names" in ckpt:
            state_dict = ckpt["optimizer"]
            saved_names = ckpt["param_names"]
            cur_names = self._get_param_names_in_optimizer_order()
            if saved_names is not None and list(saved_names) != list(cur_names):
                state_dict = _remap_optimizer_state(state_dict, saved_names, cur_names, self.optimizer)
        elif isinstance(ckpt, dict) and "optimizer" in ckpt:
            state_dict = ckpt["optimizer"]
        else:
            state_dict = ckpt  # old bare format
        self.optimizer.load_state_dict(state_dict)
        del ckpt
        gc.collect()

    def _get_param_names_in_optimizer_order(self) -> List[str]:
        names_by_id = {id(p): n for n, p in self.network.named_parameters()}
        names = []
        for group in self.optimizer.param_groups:
            for p in group["params"]:
                names.append(names_by_id.get(id(p), "?"))
        if getattr(self.optimizer, "is_fused_arena", False):
            names = self.optimizer.param_names()
        return names

    def save_optimizer(self, filename: str):
        """tmp file + rename; keeps the process alive through ctrl-c while writing"""
        print("Save optimizer under %s" % filename, file=log.v4)
        directory = os.path.dirname(filename)
        if directory:
            os.makedirs(directory, exist_ok=True)
        opts = self._optimizer_opts if isinstance(self._optimizer_opts, dict) else {}
        payload = {
            "optimizer": self.optimizer.state_dict(),
            "optimizer_class_name": type(self.optimizer).__name__,
            "optimizer_opts": {k: v for k, v in opts.items() if isinstance(v, (int, float, str, bool, type(None), list, tuple))},
            "param_names": self._get_param_names_in_optimizer_order(),
            "epoch": self._current_epoch,
            "step": self._current_train_step,
            "effective_learning_rate": self._effective_learning_rate,
            "returnn_version": _version(),
        }
        tmp = filename + ".tmp_write"
        torch.save(payload, tmp)
        os.replace(tmp, filename)

    def get_optimizer(self) -> torch.optim.Optimizer:
        """the optimizer"""
        return self.optimizer

    def _create_optimizer(self, optimizer_opts) -> torch.optim.Optimizer:
        lr = self.learning_rate
        if isinstance(optimizer_opts, torch.optim.Optimizer):
            return optimizer_opts
        if callable(optimizer_opts) and not isinstance(optimizer_opts, dict):
            return optimizer_opts(self.network.named_parameters(), lr=lr, **get_fwd_compat_kwargs())
        assert isinstance(optimizer_opts, dict), "'optimizer' must be a dict, callable or Optimizer"
        if "class" not in optimizer_opts:
            raise ValueError("'class' field of 'optimizer' dict was not set")
        opt_kwargs = optimizer_opts.copy()
        optim_class_name = opt_kwargs.pop("class")
        optim_class = get_optimizer_class(optim_class_name)
        use_fused_arena = opt_kwargs.pop("fused_arena", None)
        if "epsilon" in opt_kwargs:
            opt_kwargs["eps"] = opt_kwargs.pop("epsilon")
        if "learning_rate" in opt_kwargs or "lr" in opt_kwargs:
            raise ValueError("'learning_rate' should be set outside of the 'optimizer' dict")
        lr_mult_fn = opt_kwargs.pop("learning_rate_multiplier", None)
        # fused arena AdamW on CUDA for adam / adamw with default extras
        if optim_class in (torch.optim.AdamW, torch.optim.Adam) and self._device.type == "cuda" and use_fused_arena is not False and lr_mult_fn is None:
            from .optim.fused_adamw import FusedArenaAdamW, fused_available

            extra = set(opt_kwargs) - {"betas", "eps", "weight_decay", "weight_decay_modules_blacklist", "weight_decay_custom_include_check", "amsgrad"}
            if fused_available(self._device) and not extra and not opt_kwargs.get("amsgrad", False):
                wd_names = self._weight_decay_param_names(opt_kwargs)
                return FusedArenaAdamW(self.network, lr=lr, betas=opt_kwargs.get("betas", (0.9, 0.999)), eps=opt_kwargs.get("eps", 1e-8),
                                       weight_decay=opt_kwargs.get("weight_decay", 0.01 if optim_class is torch.optim.AdamW else 0.0),
                                       decoupled=optim_class is torch.optim.AdamW, weight_decay_param_names=wd_names, arena=self._arena)
        allowed = _get_class_init_kwargs(optim_class)
        param_groups = self._get_optimizer_param_groups(optim_class, opt_kwargs, lr_mult_fn)
        opt_kwargs.pop("weight_decay_modules_blacklist", None)
        opt_kwargs.pop("weight_decay_custom_include_check", None)
        unknown = [k for k in opt_kwargs if k not in allowed]
        if unknown and allowed:
            raise ValueError("optimizer %s: unknown options %r; allowed: %r" % (optim_class, unknown, allowed))
        optimizer = optim_class(param_groups, lr=lr, **opt_kwargs)
        print("Optimizer: %s" % optimizer.__class__.__name__, file=log.v4)
        assert isinstance(optimizer, torch.optim.Optimizer)
        return optimizer

    def _weight_decay_param_names(self, optimizer_opts: Dict[str, Any]) -> Set[str]:
        """names of the parameters which get weight decay"""
        blacklist = optimizer_opts.get("weight_decay_modules_blacklist", None)
        custom_check = optimizer_opts.get("weight_decay_custom_include_check", None)
        if blacklist is None:
            # also the option's name in the reference
            blacklist = optimizer_opts.get("weight_decay_modules_blacklist", optimizer_opts.get("blacklist_weight_decay_modules", None))
        blacklist_t = wrap_user_blacklist_wd_modules(blacklist)
        from .frontend.bridge import RFModuleAsPTModule

        wd: Set[str] = set()
        for mod_name, module in self.network.named_modules():
            rf_mod = module.rf_module if isinstance(module, RFModuleAsPTModule) else None
            for pname, param in module.named_parameters(recurse=False):
                full = "%s.%s" % (mod_name, pname) if mod_name else pname
                if custom_check is not None:
                    inc = custom_check(module=rf_mod if rf_mod is not None else module, full_param_name=full, **get_fwd_compat_kwargs())
                    if inc is not None:
                        if inc:
                            wd.add(full)
                        continue
                if pname.endswith("bias"):
                    continue
                if isinstance(module, blacklist_t) or (rf_mod is not None and isinstance(rf_mod, blacklist_t)):
                    continue
                if rf_mod is not None:
                    rp = getattr(rf_mod, pname, None)
                    if isinstance(rp, rf.Parameter) and rp.weight_decay is not None and not rp.weight_decay and False:
                        continue
                wd.add(full)
        return wd

    def _get_optimizer_param_groups(self, optim_class, optimizer_opts: Dict[str, Any], lr_mult_fn) -> List[Dict[str, Any]]:
        """param groups: weight decay yes/no, times the distinct learning rate multipliers"""
        named = [(n, p) for n, p in self.network.named_parameters() if p.requires_grad]
        allowed = _get_class_init_kwargs(optim_class)
        weight_decay = optimizer_opts.get("weight_decay", 0.0)
        if "weight_decay" not in allowed and allowed:
            weight_decay = 0.0
        groups: Dict[Tuple[bool, float], List[torch.nn.Parameter]] = {}
        wd_names = self._weight_decay_param_names(optimizer_opts) if weight_decay else set()
        for n, p in named:
            mult = 1.0
            if lr_mult_fn is not None:
                mult = float(lr_mult_fn(full_param_name=n, **get_fwd_compat_kwargs()))
            groups.setdefault((n in wd_names, mult), []).append(p)
        res = []
        for (use_wd, mult), params in groups.items():
            g: Dict[str, Any] = {"params": params}
            if weight_decay:
                g["weight_decay"] = weight_decay if use_wd else 0.0
            if mult != 1.0:
                g["learning_rate_multiplier"] = mult
            res.append(g)
        return res


def _total_norm(params) -> torch.Tensor:
    norms = torch._foreach_norm([p.grad for p in params], 2.0)
    return torch.linalg.vector_norm(torch.stack(norms), 2.0)


def _version() -> str:
    from .. import __long_version__

    return __long_version__


def _remap_optimizer_state(state_dict, saved_names, cur_names, optimizer) -> Dict[str, Any]:
    """re-index the per-parameter state by name"""
    saved_idx = {n: i for i, n in enumerate(saved_names)}
    new_state = {}
    for i, n in enumerate(cur_names):
        j = saved_idx.get(n)
        if j is not None and j in state_dict["state"]:
            new_state[i] = state_dict["state"][j]
    cur = optimizer.state_dict()
    return {"state": new_state, "param_groups": cur["param_groups"]}


def gradient_noise_(params: Iterable[torch.nn.Parameter], std: float, *, generator: Optional[torch.Generator] = None):
    """add Gaussian noise to all gradients, in place"""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    for g in grads:
        noise = torch.empty_like(g).normal_(0.0, std, generator=generator)
        g.add_(noise)


def wrap_user_blacklist_wd_modules(mods) -> Tuple[type, ...]:
    """
    The module classes whose parameters get no weight decay, from the user's option: classes, or their names as strings (``"rf.LayerNorm"``,
    ``"torch.nn.LayerNorm"``, any importable dotted name). None: norm and embedding layers of both module families.
    Parity: returnn/torch/updater.py:666.
    """
    if mods is None:
        return (rf.LayerNorm, rf.Embedding, rf.BatchNorm, torch.nn.LayerNorm, torch.nn.Embedding, torch.nn.BatchNorm1d)
    assert isinstance(mods, (list, tuple)), "invalid weight_decay_modules_blacklist %r" % (mods,)
    res = []
    for mod in mods:
        if isinstance(mod, str):
            if mod.startswith("rf."):
                mod = getattr(rf, mod[3:])
            else:
                import importlib

                mod_name, _, cls_name = mod.rpartition(".")
                mod = getattr(importlib.import_module(mod_name), cls_name)
        assert isinstance(mod, type) and issubclass(mod, (rf.Module, torch.nn.Module)), "invalid weight_decay_modules_blacklist entry %r" % (mod,)
        res.append(mod)
    return tuple(res)
