"""
Run context of one step: train flag, step/epoch, the losses marked by ``train_step`` and the outputs marked by
``forward_step``.

Loss bookkeeping: a loss tensor may have any dims; its reported value is sum(loss) / inv_norm_factor where
inv_norm_factor is the number of valid (non-padded) elements, unless ``custom_inv_norm_factor`` is given. The value
used for the gradient is ``scale * sum(loss)`` (or ``scale * mean`` with ``use_normalized_loss``). ``as_error`` entries
are reported only.

Parity: returnn/frontend/run_ctx.py:79-504 (mark_as_loss :217-288, mark_as_output :290-390, total_loss :415-426,
Loss :429-504, train_flag_ctx :129-188).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Sequence, Union
import contextlib
from ..tensor import Tensor, Dim, TensorDict, batch_dim

__all__ = ["RunCtx", "Loss", "get_run_ctx", "get_run_ctx_step", "init_train_step_run_ctx", "init_forward_step_run_ctx"]

_run_ctx: Optional["RunCtx"] = None
_init_run_ctx: Optional["RunCtx"] = None


def reset_run_ctx():
    """drop the current run ctx"""
    global _run_ctx
    _run_ctx = None


def init_train_step_run_ctx(*, train_flag: Union[bool, Tensor] = True, step: Union[int, Tensor] = 0, epoch: Union[int, Tensor] = 1):
    """new ctx for a train (or eval-with-loss) step"""
    global _run_ctx
    _run_ctx = RunCtx(stage="train_step", train_flag=train_flag, step=step, epoch=epoch)


def init_forward_step_run_ctx(*, expected_outputs: Optional[TensorDict] = None, step: Union[int, Tensor] = 0, epoch: Union[int, Tensor] = 1):
    """new ctx for a forward step"""
    global _run_ctx
    _run_ctx = RunCtx(stage="forward_step", expected_outputs=expected_outputs, step=step, epoch=epoch)


def get_run_ctx() -> "RunCtx":
    """current ctx; outside of steps, an "init" stage ctx"""
    global _init_run_ctx
    if _run_ctx is not None:
        return _run_ctx
    if _init_run_ctx is None:
        _init_run_ctx = RunCtx(stage="init")
    return _init_run_ctx


class RunCtx:
    """state of one step"""

    def __init__(self, *, stage: str, train_flag: Union[bool, Tensor] = False, step: Union[int, Tensor] = 0,
                 epoch: Union[int, Tensor] = 1, expected_outputs: Optional[TensorDict] = None):
        self._stage = stage
        self._train_flag = train_flag
        self._train_flag_per_func: Dict[Callable, bool] = {}
        self._step = step
        self._epoch = epoch
        self.losses: Dict[str, Loss] = {}
        self.outputs = TensorDict()
        self.expected_outputs = expected_outputs

    def __repr__(self):
        return "<RunCtx stage=%r train_flag=%r step=%r>" % (self._stage, self._train_flag, self._step)

    @property
    def stage(self) -> str:
        """init / train_step / forward_step"""
        return self._stage

    @property
    def train_flag(self) -> Union[bool, Tensor]:
        """dropout etc. active"""
        return self._train_flag

    @property
    def step(self) -> Union[int, Tensor]:
        """global train step"""
        return self._step

    @property
    def epoch(self) -> Union[int, Tensor]:
        """epoch"""
        return self._epoch

    def get_step_tensor(self) -> Tensor:
        """the global train step as a scalar int64 tensor (on the host)"""
        if isinstance(self._step, Tensor):
            return self._step
        import torch

        return Tensor("global_train_step", dims=(), dtype="int64", raw_tensor=torch.tensor(int(self._step), dtype=torch.int64))

    def get_epoch_tensor(self) -> Tensor:
        """the epoch as a scalar int64 tensor (on the host)"""
        if isinstance(self._epoch, Tensor):
            return self._epoch
        import torch

        return Tensor("epoch", dims=(), dtype="int64", raw_tensor=torch.tensor(int(self._epoch), dtype=torch.int64))

    def is_train_flag_enabled(self, *, func: Optional[Callable] = None) -> Union[bool, Tensor]:
        """train flag, possibly overridden for func"""
        if func is not None and func in self._train_flag_per_func:
            return self._train_flag_per_func[func]
        return self._train_flag

    @contextlib.contextmanager
    def train_flag_ctx(self, train_flag: Union[bool, Tensor], *, func: Optional[Union[Callable, Sequence[Callable]]] = None):
        """temporarily change the train flag, globally or only for the given function(s)"""
        if func is None:
            old = self._train_flag
            self._train_flag = train_flag
            try:
                yield
            finally:
                self._train_flag = old
            return
        funcs = [func] if callable(func) else list(func)
        old_per = dict(self._train_flag_per_func)
        for f in funcs:
            self._train_flag_per_func[f] = train_flag
        try:
            yield
        finally:
            self._train_flag_per_func = old_per

    def mark_as_loss(self, loss: Union[Tensor, Any], name: str, *, scale: Optional[float] = 1.0, as_error: bool = False,
                     use_normalized_loss: bool = False, use_flatten_frames: bool = True,
                     custom_inv_norm_factor: Optional[Tensor] = None) -> None:
        """register a loss; see module docstring"""
        assert self.stage == "train_step", "mark_as_loss: only inside train_step (stage %r)" % self.stage
        if not isinstance(loss, Tensor):
            from ._utils import convert_to_tensor

            loss = convert_to_tensor(loss)
        assert name not in self.losses, "mark_as_loss: duplicate loss name %r" % name
        self.losses[name] = Loss(loss=loss, name=name, scale=scale, as_error=as_error, use_normalized_loss=use_normalized_loss,
                                 use_flatten_frames=use_flatten_frames, custom_inv_norm_factor=custom_inv_norm_factor)

    def mark_as_output(self, tensor: Union[Tensor, Any], name: str, *, dims: Optional[Sequence[Dim]] = None) -> None:
        """register an output; checked against the ``model_outputs`` template when given"""
        assert self.stage == "forward_step", "mark_as_output: only inside forward_step (stage %r)" % self.stage
        expected = None
        if self.expected_outputs is not None:
            assert name in self.expected_outputs.data, "mark_as_output: unexpected output %r, we expect outputs: %s" % (
                name, self.expected_outputs)
            expected = self.expected_outputs.data[name]
        if dims is None and expected is not None:
            dims = expected.dims
        if not isinstance(tensor, Tensor):
            import torch
            import numpy
            from ._utils import convert_to_tensor

            assert dims is not None or not getattr(tensor, "ndim", 0), "mark_as_output: raw tensor %r needs dims" % name
            tensor = convert_to_tensor(tensor, dims=dims or ())
        if dims is not None:
            assert set(dims) == set(tensor.dims), "mark_as_output: %r dims %r != expected %r" % (name, tensor.dims, dims)
            if tuple(dims) != tuple(tensor.dims):
                tensor = tensor.copy_transpose_to_dims(dims)
        tensor = tensor.copy(name=name)
        if expected is not None:
            assert expected.dtype == tensor.dtype, "mark_as_output: %r dtype %s, expected %s" % (name, tensor.dtype, expected.dtype)
            assert expected.sparse_dim == tensor.sparse_dim or expected.sparse_dim is None or tensor.sparse_dim is None or (
                expected.sparse_dim.dimension == tensor.sparse_dim.dimension), "mark_as_output: %r sparse_dim %r, expected %r" % (
                name, tensor.sparse_dim, expected.sparse_dim)
            if expected.sparse_dim is not None and tensor.sparse_dim is None:
                tensor.sparse_dim = expected.sparse_dim
        assert name not in self.outputs.data, "mark_as_output: duplicate output %r" % name
        self.outputs.data[name] = tensor

    def mark_as_default_output(self, tensor: Union[Tensor, Any], *, shape: Optional[Sequence[Dim]] = None) -> None:
        """output named "output" """
        self.mark_as_output(tensor, "output", dims=shape)

    def check_outputs_complete(self):
        """all expected outputs were marked"""
        if self.expected_outputs is not None:
            for name in self.expected_outputs.data:
                assert name in self.outputs.data, "forward_step did not mark output %r" % name

    def total_loss(self) -> Union[Tensor, float]:
        """sum over scale * reduced loss of all non-error losses: the value to differentiate"""
        assert self.stage == "train_step"
        total = None
        for loss in self.losses.values():
            if loss.as_error or loss.scale is None or loss.scale == 0:
                continue
            term = loss.get_scaled_reduced_loss()
            total = term if total is None else total + term
        return 0.0 if total is None else total


class Loss:
    """one marked loss"""

    def __init__(self, *, loss: Tensor, name: str, scale=1.0, as_error=False, use_normalized_loss=False,
                 use_flatten_frames=True, custom_inv_norm_factor: Optional[Tensor] = None):
        self.loss = loss
        self.name = name
        self.scale = scale
        self.as_error = as_error
        self.use_normalized_loss = use_normalized_loss
        self.use_flatten_frames = use_flatten_frames
        self.custom_inv_norm_factor = custom_inv_norm_factor
        self._summed_loss_cached: Optional[Tensor] = None
        self._mean_loss_cached: Optional[Tensor] = None

    def get_summed_loss(self) -> Tensor:
        """sum over all valid elements, scalar"""
        if self._summed_loss_cached is not None:
            return self._summed_loss_cached
        from .reduce import reduce_sum as _reduce_sum
        from .array_ import cast

        loss = self.loss
        if not loss.dims:
            self._summed_loss_cached = loss
            return loss
        if loss.dtype == "bool" or loss.dtype.startswith("int"):
            loss = cast(loss, "float32")
        if self._mean_loss_cached is not None:
            self._summed_loss_cached = self._mean_loss_cached * self.get_inv_norm_factor()
        else:
            self._summed_loss_cached = _reduce_sum(loss, axis=loss.dims)
        return self._summed_loss_cached

    def get_mean_loss(self) -> Tensor:
        """summed / inv_norm_factor"""
        if self._mean_loss_cached is not None:
            return self._mean_loss_cached
        if self.custom_inv_norm_factor is not None or self.loss.dims:
            inv = self.get_inv_norm_factor()
            res = self.get_summed_loss() / (inv if not isinstance(inv, Tensor) else _to_device_float(inv, self.loss))
        else:
            res = self.loss
        self._mean_loss_cached = res
        return res

    def get_inv_norm_factor(self) -> Union[int, Tensor]:
        """number of valid elements (or the custom factor)"""
        if self.custom_inv_norm_factor is not None:
            f = self.custom_inv_norm_factor
            if isinstance(f, Tensor) and f.dims:
                from .reduce import reduce_sum as _reduce_sum

                f = _reduce_sum(f, axis=f.dims)
            return f
        from .array_ import num_elements_of_shape

        return num_elements_of_shape(self.loss.dims)

    def get_scaled_reduced_loss(self) -> Tensor:
        """what goes into the total loss"""
        loss = self.get_mean_loss() if self.use_normalized_loss else self.get_summed_loss()
        if self.scale != 1:
            loss = loss * self.scale
        return loss


def _to_device_float(x: Tensor, like: Tensor) -> Tensor:
    from ._utils import wrap

    raw = x._raw_tensor.to(like._raw_tensor.device)
    if not raw.is_floating_point():
        raw = raw.float()
    return wrap(raw, x._dims)


def get_run_ctx_step() -> Tensor:
    """the global train step of the current run context as a scalar tensor (``get_run_ctx().get_step_tensor()``)"""
    return get_run_ctx().get_step_tensor()
