"""
The torch engine: train / eval / forward loops around the user's ``get_model``, ``train_step`` and ``forward_step``.

Checkpoint format: ``<model>.<epoch:03d>.pt`` = ``{"model": state_dict, "epoch", "step", "effective_learning_rate",
"returnn_version"}`` and ``<model>.<epoch:03d>.opt.pt`` for the optimizer (see :mod:`returnn_b200.torch.updater`);
``step`` is the global train step *after* the epoch. Only rank 0 writes.

Per step: batch from the data loader (worker processes) -> host-to-device copy (sequence lengths stay on the host)
-> ``train_step`` under autocast -> total loss -> backward (bucketed gradient reduction overlapped) -> updater step
-> optional parameter averaging -> logging (one device-to-host read per step for all losses together).

Parity: returnn/torch/engine.py (Engine.__init__ :65-187, init_train_from_config :200-295, train :302-329,
init_train_epoch :380-415, train_epoch :462-807, eval_model :816-949, _create_data_loader :971-1054, _run_step
:1068-1128, _load_model :1130-1378, _create_model :1380-1418, _save_model :1426-1460, forward_with_callback :1496-1679,
profiler :1962-2062).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union
import contextlib
import gc
import math
import os
import re
import sys
import time
import numpy
import torch
import torch.distributed
from torch import autocast

from ..config import Config
from ..log import log
from ..engine.base import EngineBase, MODEL_POSTFIX, OPT_POSTFIX
from ..datasets.basic import Dataset, init_dataset
from ..utils.basic import hms, NumbersDict, get_fwd_compat_kwargs, BehaviorVersion
from .. import frontend as rf
from ..tensor import Tensor, Dim, TensorDict, batch_dim
from ..forward_iface import ForwardCallbackIface
from .updater import Updater
from .data import pipeline as data_pipeline
from .data import returnn_dataset_wrapper
from .data import extern_data as extern_data_util
from .frontend.bridge import rf_module_to_pt_module
from . import distributed as _distributed


class Engine(EngineBase):
    """torch engine"""

    def __init__(self, config: Config):
        super().__init__(config=config)
        rf.select_backend_torch()
        self.model_filename = self.config.value("model", None)
        self._mp_manager = None
        self._epoch_mp_shared = None
        self.train_dataset: Optional[Dataset] = None
        self.eval_datasets: Dict[str, Dataset] = {}
        self.extern_data: Optional[TensorDict] = None
        self._train_dataloader = None
        self._eval_dataloaders: Dict[str, Any] = {}
        self._start_epoch: Optional[int] = None
        self._final_epoch: Optional[int] = None
        self._min_seq_length = config.typed_value("min_seq_length", None) or config.int("min_seq_length", 0)
        self._max_seq_length = config.typed_value("max_seq_length", None) or config.int("max_seq_length", sys.maxsize)
        self._orig_model: Optional[Union[rf.Module, torch.nn.Module]] = None
        self._pt_model: Optional[torch.nn.Module] = None
        self._epoch_start_func: Optional[Callable] = self.config.typed_value("epoch_start")
        self._epoch_end_func: Optional[Callable] = self.config.typed_value("epoch_end")
        self._train_step_func: Optional[Callable] = None
        self._forward_step_func: Optional[Callable] = self.config.typed_value("forward_step")
        self._forward_step_expected_outputs = None
        if self.config.typed_value("model_outputs") is not None:
            self._forward_step_expected_outputs = TensorDict()
            self._forward_step_expected_outputs.update(self.config.typed_value("model_outputs"), auto_convert=True)
        self._save_model_epoch_interval = 1
        self._ignore_param_set: List[str] = []
        self._updater: Optional[Updater] = None
        self._use_autocast = False
        self._autocast_dtype: Optional[torch.dtype] = None
        self._grad_scaler: Optional[torch.amp.GradScaler] = None
        dev_ = get_device_from_config_opt(config.value("device", None))
        self._device = dev_.result
        print("Using device:", self._device, "(%s)" % (dev_.reason or "?"), file=log.v2)
        self._torch_distributed_ctx: Optional[_distributed.DistributedContext] = None
        self._ddp_pt_model: Optional[torch.nn.Module] = None
        if config.typed_value("torch_distributed") is not None:
            self._torch_distributed_ctx = _distributed.get_ctx(config=config)
            local_rank = self._torch_distributed_ctx.local_rank()
            print("Start running torch distributed training on local rank %i." % local_rank, file=log.v2)
            if self._device == "cuda":
                self._device = "cuda:%i" % (local_rank % max(torch.cuda.device_count(), 1))
        if self._device == "cuda":
            self._device = "cuda:%i" % torch.cuda.current_device()
        if self._device.startswith("cuda"):
            torch.cuda.set_device(self._device)
        self._log_memory_usage = config.bool("torch_log_memory_usage", False)
        self._log_batch_size = config.bool("log_batch_size", False) and log.verbose[5]
        self._calculate_exp_loss = config.bool("calculate_exp_loss", False)
        self._reset_dev_memory_caches = config.bool("reset_dev_memory_caches", False)
        self._forward_auto_split_batch_on_oom = config.bool("forward_auto_split_batch_on_oom", False)
        self._stop_on_nonfinite_train_score = config.bool("stop_on_nonfinite_train_score", True)
        self._packed_tensors = config.typed_value("packed_tensors", None)
        default_float_dtype = config.value("default_float_dtype", None)
        if default_float_dtype is not None:
            assert isinstance(default_float_dtype, str)
            rf.set_default_float_dtype(default_float_dtype)
            self._default_float_dtype = getattr(torch, default_float_dtype)
        else:
            self._default_float_dtype = None
        amp_options = self.config.opt_typed_value("torch_amp")
        grad_scaler_opts = self.config.typed_value("grad_scaler", {})
        if amp_options is not None:
            self._use_autocast = True
            if isinstance(amp_options, dict):
                amp_options = amp_options.copy()
                dtype = amp_options.pop("dtype", None)
                grad_scaler_opts = amp_options.pop("grad_scaler", grad_scaler_opts)
                assert not amp_options, "torch_amp: unknown options %r" % (amp_options,)
            elif isinstance(amp_options, str):
                dtype = amp_options
            else:
                raise TypeError("Invalid type for torch_amp: %r" % type(amp_options))
            if isinstance(dtype, str):
                dtype = getattr(torch, dtype)
            assert isinstance(dtype, torch.dtype) or dtype is None
            print("Using autocast (automatic mixed precision (AMP)) with dtype %s" % dtype, file=log.v3)
            self._autocast_dtype = dtype
        if grad_scaler_opts is None:
            self._grad_scaler = None
        elif self._use_autocast and self._autocast_dtype == torch.float16:
            self._grad_scaler = torch.amp.GradScaler(self._device.split(":")[0], **(grad_scaler_opts or {}))
        self._use_tensorboard = config.bool("use_tensorboard", False)
        self._tensorboard_writer = None
        self._tensorboard_opts = config.typed_value("tensorboard_opts", {}) or {}
        self._graph_step = None
        self._copy_stream = None  # side stream of stage_batch
        self._pending_losses = None  # (names, pinned host buffer, event) of the last step with a deferred loss read
        self._loss_slots = None
        self._epoch_mp_pending = 0
        self._nvtx = config.bool("torch_nvtx_ranges", False) and self._device.startswith("cuda")

    # -- setup -------------------------------------------------------------------------------------------------------
    def init_network_from_config(self, config: Optional[Config] = None):
        """create the model and load the checkpoint selected by the resume rules"""
        assert config is self.config or not config
        extern_data_dict = self.config.typed_value("extern_data")
        assert extern_data_dict, "extern_data is not specified in config"
        self.extern_data = extern_data_util.extern_data_template_from_config_opts(extern_data_dict)
        self._load_model()

    def init_train_from_config(self, config: Optional[Config] = None, train_data: Optional[Dataset] = None,
                               dev_data: Optional[Dataset] = None, eval_data: Optional[Dataset] = None):
        """prepare everything for ``train()``"""
        assert config is self.config or not config
        config = self.config
        super().init_train_from_config(config=config)
        self.train_dataset = train_data
        self.eval_datasets.clear()
        if dev_data:
            self.eval_datasets["dev"] = dev_data
        if eval_data:
            self.eval_datasets["eval"] = eval_data
        if config.has("eval_datasets"):
            for name, opts in config.typed_value("eval_datasets", {}).items():
                self.eval_datasets[name] = init_dataset(opts, default_kwargs={"name": name})
        self._train_dataloader = self._create_data_loader(train_data, train=True) if train_data else None
        for name, ds in self.eval_datasets.items():
            self._eval_dataloaders[name] = self._create_data_loader(ds, train=False, dataset_name=name, chunk=self.config.bool("chunk_eval", True))
        self._start_epoch = self.get_train_start_epoch(self.config)
        self._final_epoch = self.config_get_final_epoch(self.config)
        self.init_network_from_config(config=config)
        self._save_model_epoch_interval = config.int("save_interval", 1)
        self._train_step_func = self.config.typed_value("train_step")
        assert self._train_step_func, "train_step not defined"
        dist = self._torch_distributed_ctx
        if dist is not None:
            self._ddp_pt_model = dist.maybe_make_distributed_module(_WrappedModuleRunStep(module=self._pt_model, engine=self))
            dist.setup_grad_reduction(self._pt_model)
        self._updater = Updater(config=self.config, network=self._pt_model, device=torch.device(self._device),
                                initial_learning_rate=self.learning_rate)
        if dist is not None and dist.arena is not None:
            self._updater.set_arena(dist.arena)
        self._updater.create_optimizer()
        if dist is not None and dist.param_averager is not None:
            # parameter-averaging mode over NVLink: the arena optimizer runs its update inside the averaging kernel on sync steps
            self._updater.get_optimizer().param_averager = dist.param_averager
        if self._start_epoch > 1:
            self._load_optimizer()
        graph_opts = config.typed_value("torch_cuda_graph", None)
        if graph_opts:
            from .util.graph_capture import GraphCapturedTrainStep

            self._graph_step = GraphCapturedTrainStep(engine=self, opts=graph_opts if isinstance(graph_opts, dict) else {})
        self._reserve_device_memory()

    def _reserve_device_memory(self):
        """
        Batches of a length-bucketed epoch all have different shapes, and every new size class makes the caching allocator go to
        the driver (``cudaMalloc`` synchronises the device) for dozens of steps. One large block is therefore taken and returned
        to the allocator's cache up front: later requests are carved out of it without a driver call. Config
        ``torch_reserve_memory_gb``: number of GB, 0 to disable; default: a fifth of the free device memory, at most 32 GB,
        nothing on devices with less than 64 GB free.
        """
        if not str(self._device).startswith("cuda"):
            return
        want = self.config.typed_value("torch_reserve_memory_gb", None)
        try:
            free, _total = torch.cuda.mem_get_info(torch.device(self._device))
        except Exception:
            return
        if want is None:
            want = min(32.0, free / 5 / 2 ** 30) if free >= 64 * 2 ** 30 else 0.0
        nbytes = int(float(want) * 2 ** 30)
        if nbytes <= 0 or nbytes > free * 0.8:
            return
        try:
            block = torch.empty(nbytes, dtype=torch.uint8, device=self._device)
            del block
            print("Reserved %.1f GB of device memory for the allocator cache." % (nbytes / 2 ** 30), file=log.v4)
        except RuntimeError:
            pass

    # -- train -------------------------------------------------------------------------------------------------------
    def train(self):
        """all epochs"""
        assert self._pt_model is not None, "Model not initialized, call init_train_from_config()."
        assert self.train_dataset is not None, "Train dataset missing, call init_train_from_config() with train_data."
        if self._start_epoch > self._final_epoch:
            print("Already trained until final epoch %i, nothing to do." % self._final_epoch, file=log.v3)
            return
        print("Starting training at epoch %i, global train step %i" % (self._start_epoch, self.global_train_step), file=log.v3)
        self.epoch = self._start_epoch - 1
        self._check_missing_eval()
        while self.epoch + 1 <= self._final_epoch:
            self.epoch += 1
            self._epoch_mp_shared_set(self.epoch)
            self.init_train_epoch()
            self.train_epoch()
            self._maybe_stop_for_resubmission()
        print("Finished training at epoch %i, global train step %i" % (self.epoch, self.global_train_step), file=log.v3)

    def _maybe_stop_for_resubmission(self):
        if not self.config.bool("stop_for_resubmission_when_low_time_left", False):
            return
        from ..utils.basic import slurm_time_left_sec

        left = slurm_time_left_sec()
        if left is None:
            return
        factor = self.config.float("stop_for_resubmission_safety_factor", 1.5)
        epoch_time = getattr(self, "_last_epoch_duration", 0.0)
        if left < epoch_time * factor:
            print("Only %s left in the job but an epoch takes %s: stopping for resubmission." % (hms(left), hms(epoch_time)), file=log.v2)
            import signal

            os.kill(os.getpid(), signal.SIGINT)

    def _epoch_mp_shared_set(self, epoch: int):
        """the epoch that dataset workers (or the in-process data pipe) pick up at their next reset"""
        self._epoch_mp_pending = epoch  # a value created later (first data loader) starts from it
        if self._epoch_mp_shared is not None:
            self._epoch_mp_shared.value = epoch

    def init_train_epoch(self):
        """learning rate and seed for the epoch"""
        self.learning_rate = self.learning_rate_control.get_learning_rate_for_epoch(self.epoch)
        self._updater.set_learning_rate(self.learning_rate)
        self._updater.set_current_train_step(global_train_step=self.global_train_step, epoch=self.epoch, epoch_continuous=self.epoch - 1)
        self.learning_rate_control.epoch_data[self.epoch].meta.update({
            "global_train_step": self.global_train_step,
            "effective_learning_rate": self._updater.get_effective_learning_rate()})
        if self._do_save():
            self.learning_rate_control.save()
        random_seed = self.config.int("random_seed", 42)
        seed_data = [self.epoch, self.global_train_step, random_seed]
        if self._torch_distributed_ctx:
            seed_data.append(self._torch_distributed_ctx.rank())
        seed = int(numpy.random.SeedSequence(seed_data).generate_state(1)[0])
        rf.set_random_seed(seed)
        if self._epoch_start_func:
            self._epoch_start_func(epoch=self.epoch, step=self.global_train_step, model=self._orig_model, **get_fwd_compat_kwargs())

    def _maybe_reset_dev_memory_caches(self, *, force: bool = False):
        if not force and not self._reset_dev_memory_caches:
            return
        gc.collect()
        if self._device.startswith("cuda"):
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats(self._device)

    def train_epoch(self):
        """one (sub)epoch"""
        print("start", self.get_epoch_str(), "global train step", self.global_train_step, "with effective learning rate",
              self._updater.get_effective_learning_rate(), "...", file=log.v3)
        accumulated_losses_dict = NumbersDict()
        accumulated_inv_norm_factors_dict = NumbersDict()
        step_idx = 0
        epoch_start_time = time.monotonic()
        elapsed_computation_time = 0.0
        self._pt_model.train()
        self._maybe_reset_dev_memory_caches()
        # an int, or a function (epoch, epoch_continuous, global_train_step) -> int evaluated every step
        accum_grad_multiple_step_dyn = None
        accum_cfg = self.config.typed_dict.get("accum_grad_multiple_step")
        if accum_cfg is not None and not isinstance(accum_cfg, int):
            assert callable(accum_cfg), "accum_grad_multiple_step must be an int or a function"
            accum_grad_multiple_step, accum_grad_multiple_step_dyn = 0, accum_cfg
        else:
            accum_grad_multiple_step = self.config.int("accum_grad_multiple_step", 1)
        dist = self._torch_distributed_ctx
        profiler = self._make_profiler()
        total_frames = NumbersDict(0)
        total_padded = NumbersDict(0)
        data_iter = iter(self._train_dataloader)
        prefetch_iter = None
        if self.config.bool("torch_dataloader_prefetch_thread", str(self._device).startswith("cuda")):
            # batching and collation of the next batches run in a background thread while this thread issues the step
            data_iter = _PrefetchThreadIter(data_iter, depth=self.config.int("torch_dataloader_prefetch_depth", 3),
                                            pin_keys=list(self.extern_data.data.keys()) if str(self._device).startswith("cuda") else None)
            prefetch_iter = data_iter
        if str(self._device).startswith("cuda") and self.config.bool("torch_stage_batches", True):
            # the copy of batch i+1 runs on the copy stream during step i
            data_iter = self._staged_iter(data_iter)
        zero_grad_next_step = True
        cur_count_grad_accum = 0
        extern_data = None
        # per-step bookkeeping (loss values on the host, progress line, tensorboard, non-finite check). With the pipelined read
        # (default on CUDA, ``torch_deferred_loss_read``) it runs one step late, after the following step was issued.
        deferred_read = self.config.bool("torch_deferred_loss_read", str(self._device).startswith("cuda"))
        # kernels with bounded waits report through the device's status board; it is copied to pinned memory once per step and looked
        # at one step late, like the losses: no extra synchronisation, and a timed-out collective cannot go unnoticed
        from ..ops.status import StatusPoller

        status_poller = StatusPoller(self._device)
        loss_ring = None
        pending_step = None

        def finish_step(rec):
            """losses of one step reach the host here"""
            nonlocal elapsed_computation_time, accumulated_losses_dict, accumulated_inv_norm_factors_dict
            if "vals" in rec:
                host_vals = rec["vals"]
            else:
                rec["event"].synchronize()
                host_vals = rec["host"][: rec["n"]].tolist()
            names_ = rec["names"]
            losses_dict = NumbersDict({n: host_vals[i] for i, n in enumerate(names_)})
            inv_norm_factors_dict = NumbersDict()
            j = len(names_)
            for i, n in enumerate(names_):
                if rec["inv_list"][i] is not None:
                    inv_norm_factors_dict[n] = host_vals[j]
                    j += 1
                else:
                    inv_norm_factors_dict[n] = rec["static_inv"][i]
            if self._updater._log_grad_norm and rec["grad_norm"] is not None:
                losses_dict["grad_norm:p2"] = float(rec["grad_norm"])
                inv_norm_factors_dict["grad_norm:p2"] = 1.0
            step_end_time = time.monotonic()
            step_duration = step_end_time - rec["step_begin_time"]
            if "vals" not in rec:
                # the wait above belongs to the step that was issued meanwhile: count each interval once
                step_duration = step_end_time - max(rec["step_begin_time"], finish_step.last_end)
            finish_step.last_end = step_end_time
            elapsed_computation_time += step_duration
            accumulated_losses_dict += losses_dict
            accumulated_inv_norm_factors_dict += inv_norm_factors_dict
            info = losses_dict / inv_norm_factors_dict
            if self._calculate_exp_loss and info.has_values():
                extended = {}
                for key, value in info.items():
                    extended[key] = value
                    if key in rec["score_keys"]:
                        try:
                            extended[key + ":exp"] = math.exp(value)
                        except OverflowError:
                            extended[key + ":exp"] = float("inf")
                info = NumbersDict(extended)
            _print_process("ep %i train" % self.epoch, step=rec["step_idx"], eval_info=dict(info.items()), step_duration=step_duration,
                           start_elapsed=step_end_time - epoch_start_time, complete_frac=rec["complete_frac"], num_seqs=rec["num_seqs"],
                           seq_idx=rec["last_seq_idx"], log_memory_usage_device=self._device if self._log_memory_usage else None)
            if self._use_tensorboard:
                self._tb_log("train", dict(info.items()), self.global_train_step)
            if self._stop_on_nonfinite_train_score:
                if any(math.isinf(v) or math.isnan(v) for v in accumulated_losses_dict.values()):
                    self._handle_run_exception(None, extern_data=rec["extern_data"], always_direct_print=True)
                    raise Exception("Inf/nan score in step %i." % rec["step_idx"])

        finish_step.last_end = 0.0
        try:
            while True:
                with _record("data_loading", self._nvtx):
                    extern_data_raw = next(data_iter, None)
                step_begin_time = time.monotonic()
                _has_data = torch.tensor([extern_data_raw is not None], dtype=torch.int8)
                if dist:
                    dist.check_peers(self.global_train_step)  # before any collective of this step
                if dist and (step_idx == 0 or extern_data_raw is None or dist.should_sync_now(epoch_step_idx=step_idx) or dist.reduce_type != "param"):
                    torch.distributed.all_reduce(_has_data, op=torch.distributed.ReduceOp.MIN)
                if not _has_data[0]:
                    if pending_step is not None:
                        finish_step(pending_step)
                        pending_step = None
                    break
                for k, v in extern_data_raw.items():
                    if k.endswith(":seq_len"):
                        key = k[: -len(":seq_len")]
                        total_frames[key] = total_frames.get(key, 0) + int(v.sum())
                        total_padded[key] = total_padded.get(key, 0) + int(v.max()) * int(v.shape[0])
                complete_frac = float(extern_data_raw["complete_frac"]) if "complete_frac" in extern_data_raw else -1.0
                num_seqs_ = int(extern_data_raw["num_seqs"]) if "num_seqs" in extern_data_raw else -1
                last_seq_idx = int(extern_data_raw["seq_idx"].max()) if "seq_idx" in extern_data_raw else -1
                if step_idx == 0 and self._do_save() and "epoch" in extern_data_raw:
                    assert int(extern_data_raw["epoch"]) == self.epoch, "data loader epoch %i != engine epoch %i" % (int(extern_data_raw["epoch"]), self.epoch)
                self._consume_staged(extern_data_raw)
                if zero_grad_next_step and self._graph_step is None:
                    self._updater.zero_grad()
                    cur_count_grad_accum = 0
                if self._graph_step is not None:
                    # the captured step zeroes its static gradient buffers itself; everything after the replay (gradient reduction,
                    # update, parameter sync) and the per-step bookkeeping below are the same as on the eager path
                    res = self._graph_step.run_train_step_ex(extern_data_raw, dist=dist, epoch_step_idx=step_idx)
                    n_l = len(res["names"])
                    finish_step(dict(names=res["names"], inv_list=[True] * n_l, static_inv=[None] * n_l, score_keys=res["score_keys"],
                                     grad_norm=res["grad_norm"], step_idx=step_idx, step_begin_time=step_begin_time,
                                     complete_frac=complete_frac, num_seqs=num_seqs_, last_seq_idx=last_seq_idx, extern_data=None,
                                     vals=res["vals"]))
                    status_poller.step(where="train step %i" % self.global_train_step)
                    step_idx += 1
                    self.global_train_step += 1
                    ec = (self.epoch - 1 + complete_frac) if complete_frac >= 0 else ((self.epoch - 1 + (last_seq_idx + 1) / num_seqs_) if num_seqs_ > 0 else None)
                    self._updater.set_current_train_step(global_train_step=self.global_train_step, epoch=self.epoch, epoch_continuous=ec)
                    if profiler is not None:
                        profiler.step()
                        if profiler.done:
                            break
                    continue
                extern_data = extern_data_util.raw_dict_to_extern_data(
                    extern_data_raw, extern_data_template=self.extern_data, device=self._device,
                    float_dtype=self._default_float_dtype, with_eval_targets=True)
                self._run_step(extern_data, train_flag=True, train_func=True)
                train_ctx = rf.get_run_ctx()
                total_loss = train_ctx.total_loss()
                # one device-to-host read for all losses of the step
                names = list(train_ctx.losses.keys())
                summed = [train_ctx.losses[n].get_summed_loss().raw_tensor.detach().float().reshape(()) for n in names]
                inv_list = []
                for n in names:
                    f = train_ctx.losses[n].get_inv_norm_factor()
                    inv_list.append(f.raw_tensor.detach().float().reshape(()).to(summed[0].device) if isinstance(f, Tensor) else None)
                stacked = torch.stack(summed + [x for x in inv_list if x is not None]) if summed else None
                if accum_grad_multiple_step_dyn is not None:
                    accum_grad_multiple_step = int(accum_grad_multiple_step_dyn(
                        epoch=self.epoch, epoch_continuous=(self.epoch - 1 + complete_frac) if complete_frac >= 0 else None,
                        global_train_step=self.global_train_step, **get_fwd_compat_kwargs()))
                do_sync = (cur_count_grad_accum + 1) >= accum_grad_multiple_step
                if dist:
                    dist.prepare_backward(sync=do_sync)
                with _record("backward", self._nvtx):
                    ctx_mgr = self._ddp_pt_model.no_sync() if (self._ddp_pt_model is not None and not do_sync) else contextlib.nullcontext()
                    with ctx_mgr:
                        if isinstance(total_loss, Tensor) and total_loss.raw_tensor.requires_grad:
                            loss_raw = total_loss.raw_tensor  # the gradients of the accumulated steps add up (no division by their number)
                            if self._grad_scaler is not None:
                                self._grad_scaler.scale(loss_raw).backward()
                            else:
                                loss_raw.backward()
                cur_count_grad_accum += 1
                grad_norm = None
                if do_sync:
                    if dist:
                        with _record("reduce_grads", self._nvtx):
                            norm_sq = dist.maybe_reduce_grads(self._pt_model)
                            if norm_sq is not None:
                                self._updater.set_precomputed_grad_norm_sq(norm_sq)
                    with _record("optimizer_step", self._nvtx):
                        if dist:
                            dist.before_param_update(epoch_step_idx=step_idx)
                        grad_norm = self._updater.step(grad_scaler=self._grad_scaler)
                    zero_grad_next_step = True
                    if dist:
                        dist.step_after_param_update(module=self._pt_model, epoch_step_idx=step_idx)
                else:
                    zero_grad_next_step = False
                rec = dict(names=names, inv_list=inv_list, static_inv=[None if inv_list[i] is not None else float(train_ctx.losses[n].get_inv_norm_factor())
                                                                      for i, n in enumerate(names)],
                           score_keys=set(k for k, v in train_ctx.losses.items() if not v.as_error), grad_norm=grad_norm, step_idx=step_idx,
                           step_begin_time=step_begin_time, complete_frac=complete_frac, num_seqs=num_seqs_, last_seq_idx=last_seq_idx,
                           extern_data=extern_data)
                if deferred_read and stacked is not None and stacked.is_cuda:
                    # pipelined read: async copy into a pinned ring; the host waits for it after the NEXT step was issued
                    if loss_ring is None or loss_ring[0][0].numel() < stacked.numel():
                        loss_ring = [(torch.empty(max(32, stacked.numel()), dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(2)]
                    host, ev = loss_ring[step_idx % 2]
                    host[: stacked.numel()].copy_(stacked, non_blocking=True)
                    ev.record()
                    rec.update(host=host, event=ev, n=stacked.numel())
                    if pending_step is not None:
                        finish_step(pending_step)
                    pending_step = rec
                else:
                    rec["vals"] = stacked.cpu().tolist() if stacked is not None else []
                    finish_step(rec)
                status_poller.step(where="train step %i" % self.global_train_step)
                step_idx += 1
                self.global_train_step += 1
                ec = (self.epoch - 1 + complete_frac) if complete_frac >= 0 else ((self.epoch - 1 + (last_seq_idx + 1) / num_seqs_) if num_seqs_ > 0 else None)
                self._updater.set_current_train_step(global_train_step=self.global_train_step, epoch=self.epoch, epoch_continuous=ec)
                if profiler is not None:
                    profiler.step()
                    if profiler.done:
                        break
            if pending_step is not None:
                finish_step(pending_step)
                pending_step = None
            status_poller.flush(where="end of epoch %i" % self.epoch)
        except Exception as exc:
            self._handle_run_exception(exc, extern_data=extern_data)
            raise
        finally:
            if prefetch_iter is not None:
                prefetch_iter.close()
            if profiler is not None:
                profiler.finish()
        elapsed = time.monotonic() - epoch_start_time
        self._last_epoch_duration = elapsed
        elapsed_computation_percentage = elapsed_computation_time / max(elapsed, 1e-9)
        print("Trained %i steps, %s elapsed (%.1f%% computing time)" % (step_idx, hms(elapsed), elapsed_computation_percentage * 100.0), file=log.v3)
        for key in sorted(total_frames.keys()):
            if total_padded[key]:
                print("  padding ratio %s: %.1f%% of %i padded frames" % (key, 100.0 * (1.0 - total_frames[key] / total_padded[key]), total_padded[key]), file=log.v4)
        if step_idx > 0:
            accumulated_losses_dict = accumulated_losses_dict / accumulated_inv_norm_factors_dict
        accumulated_losses_dict = self._maybe_extend_losses_info(accumulated_losses_dict)
        self.learning_rate_control.epoch_data[self.epoch].meta.update({"epoch_num_train_steps": step_idx, "epoch_train_time_secs": round(elapsed)})
        self.learning_rate_control.set_epoch_error(self.epoch, {"train_loss_%s" % k: float(v) for k, v in accumulated_losses_dict.items()})
        if self._do_save():
            self.learning_rate_control.save()
        print("Total train loss:", _format_score(dict(accumulated_losses_dict.items())), file=log.v3)
        self._maybe_reset_dev_memory_caches()
        if (self.epoch % self._save_model_epoch_interval == 0) or (self.epoch == self._final_epoch):
            if self.model_filename:
                self._save_model()
                self._save_optimizer()
            else:
                print("Not saving model, `model` not specified.", file=log.v3)
        self.eval_model()
        if self.config.bool_or_other("cleanup_old_models", None):
            self.cleanup_old_models()
        if self._epoch_end_func:
            self._epoch_end_func(epoch=self.epoch, step=self.global_train_step, model=self._orig_model, **get_fwd_compat_kwargs())

    def stage_batch(self, extern_data_raw: Dict[str, Any]) -> Dict[str, Any]:
        """
        Start the host-to-device copy of a collated batch on the engine's copy stream, so that it runs while the kernels of the
        step before are still executing. The result is passed to ``run_train_step`` in place of the host batch; that call makes
        the compute stream wait for the copy. Sequence lengths and other metadata stay on the host.

        :param extern_data_raw: output of the data loader / ``collate_batch`` (pinned host tensors make the copy asynchronous)
        :return: the same dict with the data tensors on the device
        """
        if not str(self._device).startswith("cuda"):
            return extern_data_raw
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self._device)
        out = dict(extern_data_raw)
        # The device tensors come from the compute stream's pool of the caching allocator (a tensor allocated under the copy
        # stream would live in that stream's own pool, which has to grow by driver calls for every new batch shape); the copy
        # stream first waits for the compute stream as of now, so the memory's previous tenant is done with it. The step before
        # the one this batch belongs to is still executing at that point: the copy overlaps it.
        cur = torch.cuda.current_stream()
        todo = []
        for k, data in self.extern_data.data.items():
            v = extern_data_raw.get(k)
            if isinstance(v, torch.Tensor) and not v.is_cuda and data.dtype != "string":
                if not v.is_pinned():
                    v = v.pin_memory()  # a copy from pageable memory would block the host until it is done
                out[k] = torch.empty(v.shape, dtype=v.dtype, device=self._device)
                todo.append((out[k], v))
        allocated = torch.cuda.Event()
        allocated.record(cur)
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(allocated)
            for dst, src in todo:
                dst.copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
        out["_staged_event"] = ev
        return out

    @staticmethod
    def _consume_staged(extern_data_raw: Dict[str, Any]):
        """a batch from ``stage_batch``: the compute stream waits for its copy and takes over the device tensors"""
        staged_ev = extern_data_raw.get("_staged_event")
        if staged_ev is not None:
            torch.cuda.current_stream().wait_event(staged_ev)

    def _staged_iter(self, data_iter):
        """the batches of ``data_iter``, each already on its way to the device while the step before it runs"""
        prev = None
        for raw in data_iter:
            staged = self.stage_batch(raw)
            if prev is not None:
                yield prev
            prev = staged
        if prev is not None:
            yield prev

    def flush_losses(self, *, _final: bool = True) -> Dict[str, Any]:
        """
        Also looks at the kernel status words of the steps issued so far (raises ``KernelWaitTimeout`` if a bounded wait ran out).

        :return: the losses of the last step run with ``read_losses="deferred"`` that were not handed out yet ({} if none)
        """
        pending, self._pending_losses = self._pending_losses, None
        if _final and getattr(self, "_status_poller", None) is not None:
            self._status_poller.flush(where="train step %i" % (self.global_train_step - 1))
        if pending is None:
            return {}
        names, host, ev = pending
        if ev is not None:
            ev.synchronize()
        return dict(zip(names, host[: len(names)].tolist()))

    def run_train_step(self, extern_data_raw: Dict[str, Any], *, read_losses: Union[bool, str] = True) -> Dict[str, Any]:
        """
        One complete training step on one collated batch: host-to-device copy of the inputs, ``train_step`` under
        autocast, backward with the gradient reduction, optimizer update, and (``read_losses``) one device-to-host read of
        the summed losses. This is the unit that ``train_epoch`` repeats; it is public so that benchmarks and custom
        loops can drive the engine batch by batch.

        ``read_losses="deferred"`` pipelines the read: the losses of this step are copied to pinned host memory asynchronously
        and the call returns the losses of the step BEFORE (read after this step's kernels were issued, so the device never
        runs dry while the host waits); ``flush_losses()`` returns the last ones.

        :param extern_data_raw: output of the data loader / ``collate_batch`` (host tensors; pinned memory makes the copy async),
            or of ``stage_batch`` (copy already under way on the copy stream)
        :param read_losses: True, False or "deferred"
        :return: loss name -> float (``read_losses``) or device scalar tensor
        """
        dist = self._torch_distributed_ctx
        if dist:
            dist.check_peers(self.global_train_step)
        self._consume_staged(extern_data_raw)
        if self._graph_step is not None:
            # ``torch_cuda_graph``: the captured step (it zeroes its static gradients itself), then reduction and update as below
            res = self._graph_step.run_train_step_ex(extern_data_raw, dist=dist, epoch_step_idx=self.global_train_step, read=bool(read_losses))
            self.global_train_step += 1
            self._updater.set_current_train_step(global_train_step=self.global_train_step, epoch=self.epoch or 1, epoch_continuous=None)
            if getattr(self, "_status_poller", None) is None:
                from ..ops.status import StatusPoller

                self._status_poller = StatusPoller(self._device)
            self._status_poller.step(where="train step %i" % (self.global_train_step - 1))
            if res["vals"] is None:
                return {}
            return dict(zip(res["names"], res["vals"][: len(res["names"])]))
        self._updater.zero_grad()
        extern_data = extern_data_util.raw_dict_to_extern_data(
            extern_data_raw, extern_data_template=self.extern_data, device=self._device,
            float_dtype=self._default_float_dtype, with_eval_targets=True)
        self._run_step(extern_data, train_flag=True, train_func=True)
        train_ctx = rf.get_run_ctx()
        total_loss = train_ctx.total_loss()
        names = list(train_ctx.losses.keys())
        summed = [train_ctx.losses[n].get_summed_loss().raw_tensor.detach().float().reshape(()) for n in names]
        if dist:
            dist.prepare_backward(sync=True)
        loss_raw = total_loss.raw_tensor
        if self._grad_scaler is not None:
            self._grad_scaler.scale(loss_raw).backward()
        else:
            loss_raw.backward()
        if dist:
            norm_sq = dist.maybe_reduce_grads(self._pt_model)
            if norm_sq is not None:
                self._updater.set_precomputed_grad_norm_sq(norm_sq)
        if dist:
            dist.before_param_update(epoch_step_idx=self.global_train_step)
        self._updater.step(grad_scaler=self._grad_scaler)
        if dist:
            dist.step_after_param_update(module=self._pt_model, epoch_step_idx=self.global_train_step)
        self.global_train_step += 1
        self._updater.set_current_train_step(global_train_step=self.global_train_step, epoch=self.epoch or 1, epoch_continuous=None)
        if str(self._device).startswith("cuda"):
            # status words of the kernels with bounded waits: copied now, looked at after the next step was issued
            if getattr(self, "_status_poller", None) is None:
                from ..ops.status import StatusPoller

                self._status_poller = StatusPoller(self._device)
            self._status_poller.step(where="train step %i" % (self.global_train_step - 1))
        if not summed:
            return {}
        if read_losses == "deferred" and not summed[0].is_cuda:
            prev = self.flush_losses(_final=False)
            self._pending_losses = (names, torch.stack(summed).clone(), None)
            return prev
        if read_losses == "deferred":
            slot = self._loss_slots[self.global_train_step % 2] if self._loss_slots else None
            if slot is None or slot[0].numel() < len(names):
                self._loss_slots = [(torch.empty(max(16, len(names)), dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(2)]
                slot = self._loss_slots[self.global_train_step % 2]
            host, ev = slot
            host[: len(names)].copy_(torch.stack(summed), non_blocking=True)
            ev.record()
            prev = self.flush_losses(_final=False)  # waits for the step before this one; this step's kernels are queued already
            self._pending_losses = (names, host, ev)
            return prev
        if read_losses:
            vals = torch.stack(summed).cpu().tolist()
            return dict(zip(names, vals))
        return dict(zip(names, summed))

    def _maybe_extend_losses_info(self, losses: NumbersDict) -> NumbersDict:
        if self._calculate_exp_loss and losses.has_values():
            ctx = rf.get_run_ctx()
            score_keys = set(k for k, v in ctx.losses.items() if not v.as_error) if ctx.stage == "train_step" else set(losses.keys())
            losses_ = {}
            for key, value in losses.items():
                losses_[key] = value
                if key in score_keys:
                    try:
                        losses_[key + ":exp"] = math.exp(value)
                    except OverflowError:
                        losses_[key + ":exp"] = float("inf")
            losses = NumbersDict(losses_)
        return losses

    def _check_missing_eval(self):
        """if a previous run saved a model but was interrupted before the evaluation of that epoch: redo it"""
        if not self.learning_rate_control or not self.eval_datasets or self.epoch <= 0:
            return
        if not self.learning_rate_control.need_error_info:
            return
        if self.epoch in self.learning_rate_control.epoch_data:
            missing = [name for name in self.eval_datasets if not self._is_dataset_evaluated(name)]
            if missing and self.epoch % self._save_model_epoch_interval == 0:
                print("Last epoch model not yet evaluated on %s. Doing that now." % ", ".join(missing), file=log.v3)
                self.eval_model(skip_already_evaluated=True)

    def eval_model(self, *, skip_already_evaluated: bool = False):
        """run ``train_step`` without update on all eval datasets; rank 0 evaluates, the others wait"""
        self._pt_model.eval()
        self._maybe_reset_dev_memory_caches()
        eval_dump_str = []
        score_keys = None
        error_keys = None
        dist = self._torch_distributed_ctx
        is_main = (not dist) or dist.rank() == 0
        for dataset_name, dataset in self.eval_datasets.items():
            if skip_already_evaluated and self._is_dataset_evaluated(name=dataset_name):
                continue
            if not is_main:
                continue
            data_loader = self._eval_dataloaders[dataset_name]
            self._epoch_mp_shared_set(self.epoch)
            print("Evaluating dataset %r" % dataset_name, file=log.v3)
            accumulated_losses_dict = NumbersDict()
            accumulated_inv_norm_factors_dict = NumbersDict()
            step_idx = 0
            eval_start_time = time.monotonic()
            with torch.no_grad():
                for extern_data_raw in data_loader:
                    step_begin_time = time.monotonic()
                    extern_data = extern_data_util.raw_dict_to_extern_data(
                        extern_data_raw, extern_data_template=self.extern_data, device=self._device,
                        float_dtype=self._default_float_dtype, with_eval_targets=True)
                    self._run_step(extern_data, train_func=True)
                    train_ctx = rf.get_run_ctx()
                    if score_keys is None:
                        score_keys = [k for k, v in train_ctx.losses.items() if not v.as_error]
                        error_keys = [k for k, v in train_ctx.losses.items() if v.as_error]
                    losses_dict = NumbersDict({name: float(loss.get_summed_loss().raw_tensor.detach().cpu()) for name, loss in train_ctx.losses.items()})
                    inv_norm = NumbersDict({name: float(_to_host(loss.get_inv_norm_factor())) for name, loss in train_ctx.losses.items()})
                    accumulated_losses_dict += losses_dict
                    accumulated_inv_norm_factors_dict += inv_norm
                    step_end = time.monotonic()
                    _print_process("ep %i %s eval" % (self.epoch, dataset_name), step=step_idx,
                                   eval_info=dict(self._maybe_extend_losses_info(losses_dict / inv_norm).items()),
                                   step_duration=step_end - step_begin_time, start_elapsed=step_end - eval_start_time, log_memory_usage_device=None)
                    step_idx += 1
            assert step_idx > 0, "No data in dataset %r." % dataset_name
            accumulated_losses_dict = accumulated_losses_dict / accumulated_inv_norm_factors_dict
            accumulated_losses_dict = self._maybe_extend_losses_info(accumulated_losses_dict)
            self.learning_rate_control.set_epoch_error(self.epoch, {"%s_loss_%s" % (dataset_name, k): float(v) for k, v in accumulated_losses_dict.items()})
            if self._do_save():
                self.learning_rate_control.save()
            eval_dump_str.append("%s: %s" % (dataset_name, _format_score(dict(accumulated_losses_dict.items()))))
            if self._use_tensorboard:
                self._tb_log(dataset_name, dict(accumulated_losses_dict.items()), self.global_train_step)
        if dist and dist.size() > 1 and self.eval_datasets:
            # epoch scores go out from rank 0 so that every rank takes the same learning-rate decisions
            obj = [self.learning_rate_control.epoch_data.get(self.epoch)] if is_main else [None]
            torch.distributed.broadcast_object_list(obj, src=0)
            if not is_main and obj[0] is not None:
                self.learning_rate_control.epoch_data[self.epoch] = obj[0]
        if not self._torch_distributed_ctx or self._torch_distributed_ctx.rank() == 0:
            print("Epoch %i evaluation:" % self.epoch, " ".join(eval_dump_str) if eval_dump_str else "(No evaluations.)", file=log.v1)
        self._maybe_reset_dev_memory_caches()

    # -- data loader -------------------------------------------------------------------------------------------------
    def _create_data_loader(self, dataset: Dataset, *, train: bool = False, dataset_name: Optional[str] = None, dataset_init_epoch: bool = True,
                            chunk: Optional[bool] = None):
        """dataset -> pipes -> DataLoader"""
        loader_opts = dict(self.config.typed_value("torch_dataloader_opts") or {})
        num_workers = loader_opts.get("num_workers", 0)
        if num_workers and self._epoch_mp_shared is None:
            from ..utils.multi_proc_manager_with_watchdog import create_manager

            self._mp_manager = create_manager()
            self._epoch_mp_shared = self._mp_manager.Value("i", self._epoch_mp_pending)
        if self._epoch_mp_shared is None:
            self._epoch_mp_shared = _LocalValue(self._epoch_mp_pending)
        if not dataset_init_epoch:
            reset_cb = returnn_dataset_wrapper.ReturnnDatasetResetNoOpCallback()
        else:
            reset_cb = returnn_dataset_wrapper.ReturnnDatasetResetMpSharedEpochCallback(dataset=dataset, epoch_mp_shared=self._epoch_mp_shared)
        wrapped = returnn_dataset_wrapper.ReturnnDatasetIterDataPipe(dataset, reset_callback=reset_cb)
        if (self._min_seq_length and self._min_seq_length != 0) or (self._max_seq_length and self._max_seq_length != sys.maxsize):
            wrapped = data_pipeline.LenFilterDataPipe(wrapped, min_seq_length=self._min_seq_length, max_seq_length=self._max_seq_length)
        chunking = self.config.typed_value("chunking", None)
        min_chunk_size = self.config.typed_value("min_chunk_size", 0)
        # training data is chunked; the evaluation data sets of a training run as well (as in the reference, so that their scores are
        # comparable with the training scores; ``chunk_eval = False`` scores whole sequences); forward / search never
        if chunking and (train if chunk is None else chunk):
            wrapped = data_pipeline.ChunkingIterDataPipe(wrapped, chunking, min_chunk_size=min_chunk_size)
        batches = data_pipeline.get_batching_iterable_dataset_from_config(dataset=wrapped, config=self.config, train=train)
        online_shuffle_batches = self.config.typed_value("online_shuffle_batches", None)
        if train and online_shuffle_batches:
            if isinstance(online_shuffle_batches, int):
                online_shuffle_batches = {"buffer_size": online_shuffle_batches}
            batches = data_pipeline.ShufflingDataPipe(batches, monotonic_data_keys=("complete_frac", "seq_idx"), **online_shuffle_batches)
        packing = None
        if self._packed_tensors:
            packing = self._packed_tensors if isinstance(self._packed_tensors, dict) else {"keys": None}
        return data_pipeline.create_data_loader_from_batches(batches, loader_opts, packing=packing)

    # -- step --------------------------------------------------------------------------------------------------------
    def _run_step(self, extern_data: TensorDict, *, train_flag: bool = False, train_func: bool, _inside_wrapped: bool = False):
        """one ``train_step`` or ``forward_step`` call under autocast with a fresh run ctx"""
        if self._ddp_pt_model is not None and not _inside_wrapped:
            self._ddp_pt_model(extern_data=extern_data, train_flag=train_flag, train_func=train_func)
            return
        if train_func:
            assert self._train_step_func is not None
            rf.init_train_step_run_ctx(train_flag=train_flag, step=self.global_train_step, epoch=self.epoch)
        else:
            assert self._forward_step_func is not None, "define forward_step in the config"
            rf.init_forward_step_run_ctx(expected_outputs=self._forward_step_expected_outputs, step=self.global_train_step, epoch=self.epoch)
        with (autocast(device_type=self._device.split(":")[0], dtype=self._autocast_dtype) if self._use_autocast else contextlib.nullcontext()), \
                rf.set_default_device_ctx(self._device), _record("model_step", self._nvtx):
            sentinel_kw = get_fwd_compat_kwargs()
            if train_func:
                self._train_step_func(model=self._orig_model, extern_data=extern_data, **sentinel_kw)
            else:
                self._forward_step_func(model=self._orig_model, extern_data=extern_data, **sentinel_kw)

    # -- model create / load / save ----------------------------------------------------------------------------------
    def _load_model(self):
        """resume rules + ``preload_from_files``"""
        checkpoint_state = None
        epoch, model_epoch_filename = self.get_epoch_model(self.config)
        step = None
        filename = None
        if model_epoch_filename:
            filename = model_epoch_filename + MODEL_POSTFIX if not os.path.exists(model_epoch_filename) or os.path.isdir(model_epoch_filename) else model_epoch_filename
            print("Load model %s" % filename, file=log.v4)
            checkpoint_state = _torch_load(filename, device=self._device)
            if epoch is None:
                epoch = checkpoint_state.get("epoch", self._start_epoch or 1)
            step = checkpoint_state.get("step", 1)
            print("  epoch %i, global train step %i" % (epoch, step), file=log.v4)
            # the stored step is the first step of the next epoch
            step -= 1
        is_training = self.config.value("task", "train") == "train"
        is_first_train_epoch = not epoch and (is_training or self.config.value("task", "train") == "initialize_model")
        if not model_epoch_filename:
            epoch = self._start_epoch or 1
            step = 0
        self._create_model(epoch=epoch, step=step)
        if checkpoint_state is not None:
            sd = checkpoint_state.get("model", checkpoint_state)
            missing_keys, unexpected_keys = self._pt_model.load_state_dict(sd, strict=False)
            missing_keys = [k for k in missing_keys if not self._is_non_critical(k)]
            if missing_keys:
                raise Exception("\n".join([
                    "While loading model %s:" % filename,
                    "Unexpected key(s) in state_dict: " + ", ".join(map(repr, unexpected_keys)),
                    "Missing key(s) in state_dict: " + ", ".join(map(repr, missing_keys)),
                    "Any missing key is an error."]))
            if unexpected_keys:
                print("Note: While loading %s, unexpected key(s) in state_dict: %s" % (filename, ", ".join(map(repr, unexpected_keys))), file=log.v4)
        preload_from_files = self.config.typed_value("preload_from_files", {}) or {}
        if preload_from_files:
            self._preload_from_files(preload_from_files, is_first_train_epoch=is_first_train_epoch, is_training=is_training)
        if self._default_float_dtype:
            self._pt_model.to(dtype=self._default_float_dtype)
        self._pt_model.to(self._device)
        for hook in self.config.typed_value("load_model_post_hooks", None) or []:
            hook(model=self._orig_model, **get_fwd_compat_kwargs())
        if model_epoch_filename and is_training:
            epoch += 1
            step += 1
        self.epoch = epoch
        self.global_train_step = step

    def _is_non_critical(self, key: str) -> bool:
        if isinstance(self._orig_model, rf.Module):
            try:
                p = self._orig_model.get_deep(key)
                return bool(getattr(p, "non_critical_for_restore", False))
            except Exception:
                return False
        return False

    def _preload_from_files(self, preload_from_files: Dict[str, Any], *, is_first_train_epoch: bool, is_training: bool):
        """
        ``{name: {"filename": ..., "prefix": "", "init_for_train": False, "ignore_missing": False, "ignore_params": (),
        "ignore_params_prefixes": (), "var_name_mapping": {}, "custom_missing_load_func": fn, "checkpoint_key": "model",
        "pattern": regex}}``
        """
        loaded_state_keys = set()
        for preload_key, opts in sorted(preload_from_files.items()):
            opts = dict(opts)
            init_for_train = opts.pop("init_for_train", False)
            if init_for_train == "always":
                pass
            elif init_for_train:
                if not (is_training and is_first_train_epoch):
                    continue
            else:
                if is_training:
                    continue
            filename = opts.pop("filename")
            print("Pre-load weights for key %r from %s" % (preload_key, filename), file=log.v3)
            state = _torch_load(filename, device=self._device)
            ckpt_key = opts.pop("checkpoint_key", "model")
            if ckpt_key is not None and ckpt_key in state:
                state = state[ckpt_key]
            ignore_params = set(opts.pop("ignore_params", ()))
            ignore_prefixes = tuple(opts.pop("ignore_params_prefixes", ()))
            state = {k: v for k, v in state.items() if k not in ignore_params and not (ignore_prefixes and k.startswith(ignore_prefixes))}
            mapping = opts.pop("var_name_mapping", {})
            if mapping:
                state = {mapping.get(k, k): v for k, v in state.items()}
            pattern = opts.pop("pattern", None)
            if pattern:
                state = {k: v for k, v in state.items() if re.match(pattern, k)}
            prefix = opts.pop("prefix", "")
            prefix_keys = [k for k in self._pt_model.state_dict() if k.startswith(prefix)]
            custom_missing = opts.pop("custom_missing_load_func", None)
            if custom_missing:
                for key in prefix_keys:
                    if key[len(prefix):] not in state:
                        cur = self._pt_model.state_dict()[key]
                        val = custom_missing(name=key[len(prefix):], shape=cur.shape, preload_model_state=state, **get_fwd_compat_kwargs())
                        if val is not None:
                            state[key[len(prefix):]] = torch.as_tensor(val) if not isinstance(val, torch.Tensor) else val
            ignore_missing = opts.pop("ignore_missing", False)
            assert not opts, "preload_from_files[%r]: unknown options %r" % (preload_key, opts)
            state = {prefix + k: v for k, v in state.items()}
            missing, unexpected = self._pt_model.load_state_dict(state, strict=False)
            loaded_state_keys.update(state.keys())
            missing_in_prefix = [k for k in missing if k in prefix_keys and not self._is_non_critical(k)]
            if missing_in_prefix and not ignore_missing:
                raise Exception("preload_from_files[%r] %s: missing keys %r (prefix %r)" % (preload_key, filename, missing_in_prefix, prefix))
            if unexpected:
                print("  note: unexpected keys (ignored): %s" % ", ".join(unexpected[:10]), file=log.v4)

    def _create_model(self, *, epoch: int, step: int):
        """seed, then the user's ``get_model``"""
        random_seed = self.config.int("random_seed", 42)
        random_seed = (epoch * 193939 + step * 19937 + random_seed * 27644437 + 479001599) % (2 ** 31)
        rf.set_random_seed(random_seed)
        get_model_func = self.config.typed_value("get_model")
        assert get_model_func, "get_model not defined in config"
        with rf.set_default_device_ctx(None):
            model = get_model_func(epoch=epoch, step=step, device=self._device, **get_fwd_compat_kwargs())
        self._orig_model = model
        if isinstance(model, rf.Module):
            self._pt_model = rf_module_to_pt_module(model)
        elif isinstance(model, torch.nn.Module):
            self._pt_model = model
        else:
            raise TypeError("get_model returned %r, expected rf.Module or torch.nn.Module" % type(model))
        assert isinstance(self._pt_model, torch.nn.Module)
        print("Model:", self._pt_model.__class__.__name__, file=log.v4)
        num_params = sum(p.numel() for p in self._pt_model.parameters())
        print("net params #:", num_params, file=log.v2)

    def get_pt_model(self) -> Optional[torch.nn.Module]:
        """the torch module"""
        return self._pt_model

    def _save_model(self):
        """write ``<model>.<epoch>.pt`` (rank 0 only; tmp file + rename)"""
        if not self._do_save():
            return
        filename = self.get_epoch_model_filename() + MODEL_POSTFIX
        directory = os.path.dirname(filename)
        if directory:
            os.makedirs(directory, exist_ok=True)
        print("Save model under %s" % filename, file=log.v4)
        tmp = filename + ".tmp_write"
        if os.path.exists(tmp):
            os.unlink(tmp)
        from .. import __long_version__

        torch.save({"model": self._pt_model.state_dict(), "epoch": self.epoch, "step": self.global_train_step,
                    "effective_learning_rate": self._updater.get_effective_learning_rate() if self._updater else None,
                    "returnn_version": __long_version__}, tmp)
        os.replace(tmp, filename)

    def get_pt_optimizer(self) -> Optional[torch.optim.Optimizer]:
        """the optimizer"""
        return self._updater.get_optimizer() if self._updater else None

    def _load_optimizer(self):
        """optimizer state of the epoch before the start epoch"""
        filename = self.get_epoch_model_filename(epoch=self._start_epoch - 1) + OPT_POSTFIX
        self._updater.load_optimizer(filename)

    def _save_optimizer(self):
        """write the optimizer file; keep only the last two"""
        if not self._do_save():
            return
        filename = self.get_epoch_model_filename() + OPT_POSTFIX
        self._updater.save_optimizer(filename)
        clean_epoch = self.epoch - 2 * self._save_model_epoch_interval
        apply_keep_logic = self.config.bool("apply_cleanup_old_models_to_optim_states", False)
        if clean_epoch > 0 and not apply_keep_logic:
            old = self.get_epoch_model_filename(epoch=clean_epoch) + OPT_POSTFIX
            if os.path.isfile(old):
                os.unlink(old)

    # -- forward -----------------------------------------------------------------------------------------------------
    def forward_with_callback(self, *, dataset: Dataset, callback: ForwardCallbackIface, dataset_init_epoch: bool = True, allow_skipping_seqs: bool = False):
        """run ``forward_step`` over the dataset; every sequence's outputs go to ``callback.process_seq``"""
        assert isinstance(dataset, Dataset) and isinstance(callback, ForwardCallbackIface)
        self._pt_model.eval()
        self._maybe_reset_dev_memory_caches()
        if dataset_init_epoch:
            if not self._min_seq_length and self._max_seq_length == sys.maxsize and dataset.supports_seq_order_sorting():
                print("Dataset supports sorting, i.e. it will be sorted for optimal performance.", file=log.v3)
                dataset.seq_ordering = "sorted_reverse"
            else:
                print("Dataset does not support sorting.", file=log.v3)
            assert (self._min_seq_length == 0 or not self._min_seq_length) and self._max_seq_length == sys.maxsize or allow_skipping_seqs or self.config.bool("allow_skipping_seqs_in_forward", False), (
                "min_seq_length / max_seq_length would skip sequences in forward; set allow_skipping_seqs_in_forward")
        self._epoch_mp_shared_set(self.epoch or 1)
        data_loader = self._create_data_loader(dataset, dataset_init_epoch=dataset_init_epoch)
        batch_dim_ = batch_dim
        pending: List[Dict[str, Any]] = []
        data_iter = iter(data_loader)

        def next_batch():
            if pending:
                return pending.pop(0)
            return next(data_iter, None)

        epoch_start_time = time.monotonic()
        step_idx = 0
        with torch.no_grad():
            callback.init(model=self._orig_model)
            while True:
                extern_data_raw = next_batch()
                if extern_data_raw is None:
                    break
                step_begin = time.monotonic()
                try:
                    extern_data = extern_data_util.raw_dict_to_extern_data(
                        extern_data_raw, extern_data_template=self.extern_data, device=self._device, float_dtype=self._default_float_dtype)
                    self._run_step(extern_data, train_func=False)
                    ctx = rf.get_run_ctx()
                    ctx.check_outputs_complete()
                    outputs = ctx.outputs
                except RuntimeError as exc:
                    if self._forward_auto_split_batch_on_oom and _is_oom(exc) and extern_data_util.raw_dict_can_split_batch(extern_data_raw):
                        print("Out of memory in forward, splitting the batch in two and retrying: %s" % str(exc).splitlines()[0], file=log.v3)
                        del exc
                        gc.collect()
                        if self._device.startswith("cuda"):
                            torch.cuda.empty_cache()
                        pending[:0] = extern_data_util.raw_dict_split_batch(extern_data_raw, splits=2)
                        continue
                    raise
                seq_tags = extern_data_raw["seq_tag"]
                n = len(seq_tags)
                host = {}
                for k, v in outputs.data.items():
                    raw = v.raw_tensor
                    host[k] = raw.detach().cpu() if isinstance(raw, torch.Tensor) else raw
                size_cache: Dict[int, Any] = {}
                for b in range(n):
                    seq_outputs = TensorDict()
                    for k, v in outputs.data.items():
                        seq_outputs.data[k] = _slice_seq(v, host[k], b, size_cache)
                    callback.process_seq(seq_tag=str(seq_tags[b]), outputs=seq_outputs)
                step_end = time.monotonic()
                _print_process("ep %i forward" % (self.epoch or 0), step=step_idx, eval_info=None, step_duration=step_end - step_begin,
                               start_elapsed=step_end - epoch_start_time,
                               complete_frac=float(extern_data_raw["complete_frac"]) if "complete_frac" in extern_data_raw else -1,
                               log_memory_usage_device=self._device if self._log_memory_usage else None)
                step_idx += 1
            callback.finish()
        print("Forward %i steps, %s elapsed" % (step_idx, hms(time.monotonic() - epoch_start_time)), file=log.v3)
        self._maybe_reset_dev_memory_caches()

    def analyze(self, data: Dataset, statistics: Optional[List[str]] = None) -> Dict[str, Any]:
        """task ``analyze``: statistics of the model's per-frame class distribution over ``data`` (see :mod:`.serving`)"""
        from .serving import analyze

        return analyze(self, data, statistics)

    def web_server(self, port: Optional[int] = None):
        """task ``search_server``: serve ``forward_step`` over HTTP until interrupted (see :mod:`.serving`)"""
        from .serving import ModelServer

        cfg = self.config
        server = ModelServer(self, port=port if port is not None else cfg.int("web_server_port", 12380), host=cfg.value("web_server_host", "127.0.0.1"),
                             max_batch=cfg.int("web_server_max_batch", 16), batch_wait_ms=cfg.float("web_server_batch_wait_ms", 2.0))
        server.serve_forever()

    # -- misc --------------------------------------------------------------------------------------------------------
    def _handle_run_exception(self, exc: Optional[Exception], *, extern_data=None, always_direct_print: bool = False):
        from .util import diagnose_gpu

        print("%s while running step %i of epoch %i." % (type(exc).__name__ if exc else "Problem", self.global_train_step, self.epoch), file=log.v1)
        if extern_data is not None:
            try:
                tags = extern_data.data.get("seq_tag")
                if tags is not None:
                    print("  seq tags: %s" % list(tags.raw_tensor)[:10], file=log.v1)
            except Exception:
                pass
        if exc is not None and self._device.startswith("cuda") and _is_oom(exc):
            diagnose_gpu.garbage_collect()
            print(torch.cuda.memory_summary(self._device, abbreviated=True), file=log.v3)

    def _make_profiler(self):
        opts = self.config.typed_value("torch_profile", None)
        if not opts:
            return None
        if self._torch_distributed_ctx and self._torch_distributed_ctx.rank() != 0:
            return None
        return _TorchProfilerCtx(opts if isinstance(opts, dict) else {})

    def _tb_log(self, prefix: str, values: Dict[str, float], step: int):
        every = self._tensorboard_opts.get("log_every_n_train_steps", 100)
        if prefix == "train" and step % every != 0:
            return
        if self._tensorboard_writer is None:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self._tensorboard_writer = SummaryWriter(**{k: v for k, v in self._tensorboard_opts.items() if k != "log_every_n_train_steps"})
            except Exception as exc:
                print("tensorboard not available (%s), disabling" % exc, file=log.v2)
                self._use_tensorboard = False
                return
        for k, v in values.items():
            self._tensorboard_writer.add_scalar("%s/%s" % (prefix, k), v, global_step=step)


class _PrefetchThreadIter:
    """
    Iterator over a data loader that runs ``next()`` (dataset access, batching, collation) and the copy into pinned host memory
    in a background thread, ``depth`` batches ahead. The collation of a 40k-frame batch takes a few milliseconds of mostly
    GIL-free tensor work; on the main thread it would be added to the time the host needs to issue a step. Exceptions of the
    producer are re-raised by the consumer. The thread ends with the iterator (end of data, ``close()`` or garbage collection).
    """

    _END = object()

    def __init__(self, it, *, depth: int = 3, pin_keys: Optional[List[str]] = None):
        import queue
        import threading

        self._it = it
        self._pin_keys = pin_keys
        self._queue: "queue.Queue" = queue.Queue(maxsize=max(1, depth))
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._produce, name="train-data-prefetch", daemon=True)
        self._thread.start()

    def _put(self, item) -> bool:
        import queue

        while not self._stop.is_set():
            try:
                self._queue.put(item, timeout=0.1)
                return True
            except queue.Full:
                continue
        return False

    def _produce(self):
        try:
            for raw in self._it:
                if self._pin_keys is not None:
                    for k in self._pin_keys:
                        v = raw.get(k)
                        if isinstance(v, torch.Tensor) and not v.is_cuda and not v.is_pinned():
                            raw[k] = v.pin_memory()
                if not self._put(raw):
                    return
            self._put(self._END)
        except BaseException as exc:  # handed to the consumer
            self._put(exc)

    def __iter__(self):
        return self

    def __next__(self):
        item = self._queue.get()
        if item is self._END:
            self._stop.set()
            raise StopIteration
        if isinstance(item, BaseException):
            self._stop.set()
            raise item
        return item

    def close(self):
        """stop the producer"""
        self._stop.set()

    def __del__(self):
        self._stop.set()


class _LocalValue:
    """same interface as a multiprocessing Value, for the single-process case"""

    def __init__(self, value):
        self.value = value


def _to_host(x) -> float:
    if isinstance(x, Tensor):
        return float(x.raw_tensor.detach().cpu())
    return float(x)


def _slice_seq(template: Tensor, host_raw, b: int, size_cache: Dict[int, Any]) -> Tensor:
    """entry b of a batched output as numpy, padding cut away"""
    dims = list(template.dims)
    if batch_dim not in dims:
        arr = host_raw.numpy() if isinstance(host_raw, torch.Tensor) and host_raw.dtype != torch.bfloat16 else (host_raw.float().numpy() if isinstance(host_raw, torch.Tensor) else host_raw)
        t = template.copy_template()
        t._raw_tensor = arr
        return t
    bax = dims.index(batch_dim)
    raw = host_raw.select(bax, b) if isinstance(host_raw, torch.Tensor) else numpy.take(host_raw, b, axis=bax)
    out_dims = dims[:bax] + dims[bax + 1:]
    new_dims = []
    for i, d in enumerate(out_dims):
        if d.is_dynamic() and d.dyn_size_ext is not None and d.dyn_size_ext.dims and batch_dim in d.dyn_size_ext.dims:
            key = id(d.get_same_base())
            if key not in size_cache:
                size_cache[key] = d.dyn_size_ext.raw_tensor.cpu() if isinstance(d.dyn_size_ext.raw_tensor, torch.Tensor) else d.dyn_size_ext.raw_tensor
            n = int(size_cache[key][b])
            raw = raw.narrow(i, 0, n) if isinstance(raw, torch.Tensor) else numpy.take(raw, range(n), axis=i)
            nd = Dim(None, name=d.name)
            nd.dyn_size_ext = Tensor("%s:size" % d.name, dims=[], dtype="int32", raw_tensor=torch.tensor(n, dtype=torch.int32))
            new_dims.append(nd)
        else:
            new_dims.append(d)
    if isinstance(raw, torch.Tensor):
        raw = (raw.float() if raw.dtype == torch.bfloat16 else raw).numpy()
    t = Tensor(template.name, dims=new_dims, dtype=str(raw.dtype), sparse_dim=template.sparse_dim)
    t._raw_tensor = raw
    return t


def _is_oom(exc: BaseException) -> bool:
    if isinstance(exc, torch.cuda.OutOfMemoryError):
        return True
    return "out of memory" in str(exc).lower()


def _torch_load(filename: str, *, device: str) -> Dict[str, Any]:
    if filename.endswith(".safetensors"):
        from safetensors.torch import load_file

        return {"model": load_file(filename, device=device)}
    return torch.load(filename, map_location=device, weights_only=False)


class _Result:
    def __init__(self, result: str, reason: Optional[str] = None):
        self.result = result
        self.reason = reason


def get_device_from_config_opt(device: Optional[str]) -> _Result:
    """``device`` config value (None / "gpu" / "cuda" / "cpu" / "cuda:1") -> torch device string"""
    if os.environ.get("PT_DEVICE"):
        return _Result(os.environ["PT_DEVICE"], "PT_DEVICE env var")
    if not device:
        if torch.cuda.is_available():
            return _Result("cuda", "'device' in config not set, CUDA is available")
        return _Result("cpu", "'device' in config not set, CUDA not available")
    if device == "gpu":
        if not torch.cuda.is_available():
            from .util import diagnose_gpu

            raise Exception("No GPU device found, but config requested 'gpu' device.\n" + "\n".join(diagnose_gpu.diagnose_no_gpu()))
        return _Result("cuda", "'gpu' in config")
    return _Result(device, "config")


@contextlib.contextmanager
def _record(name: str, nvtx: bool):
    if nvtx:
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.autograd.profiler.record_function(name):
            yield
    finally:
        if nvtx:
            torch.cuda.nvtx.range_pop()


class _TorchProfilerCtx:
    """``torch_profile`` config: profile some steps on rank 0, export a Chrome trace, then stop"""

    def __init__(self, opts: Dict[str, Any]):
        from torch.profiler import profile, ProfilerActivity, schedule

        opts = dict(opts)
        self.trace_file = opts.pop("trace_file", "torch_profile.json")
        sched = dict(skip_first=10, wait=5, warmup=3, active=3, repeat=1)
        sched.update(opts.pop("schedule", {}))
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self.total_steps = sched["skip_first"] + sched["wait"] + sched["warmup"] + sched["active"]
        self.prof = profile(activities=acts, schedule=schedule(**sched), record_shapes=opts.pop("record_shapes", False),
                            profile_memory=opts.pop("profile_memory", False), with_stack=opts.pop("with_stack", False))
        self.prof.__enter__()
        self.n = 0
        self.done = False

    def step(self):
        """after each train step"""
        self.prof.step()
        self.n += 1
        if self.n >= self.total_steps:
            self.done = True

    def finish(self):
        """export"""
        self.prof.__exit__(None, None, None)
        try:
            self.prof.export_chrome_trace(self.trace_file)
            print("Wrote profile trace to %s" % self.trace_file, file=log.v2)
        except Exception as exc:
            print("Could not export profile trace: %s" % exc, file=log.v2)


class _WrappedModuleRunStep(torch.nn.Module):
    """
    A module whose forward runs the whole user step; this is what a user-given DDP-like ``class`` wraps, so that its
    forward/backward hooks see the step.
    """

    def __init__(self, *, module: torch.nn.Module, engine: Engine):
        super().__init__()
        self.module = module
        self.engine = engine

    def forward(self, *args, **kwargs):
        """one step; returns the total loss so that wrappers that inspect outputs see a tensor"""
        self.engine._run_step(*args, **kwargs, _inside_wrapped=True)
        if rf.get_run_ctx().stage == "train_step":
            total = rf.get_run_ctx().total_loss()
            return total.raw_tensor if isinstance(total, Tensor) else total
        return None


def _format_score(score: Dict[str, float]) -> str:
    if not score:
        return "None"
    if len(score) == 1:
        return "%.3f" % float(list(score.values())[0])
    return " ".join("%s %.3f" % (k, v) for k, v in score.items())


_last_print_time = [0.0]


def _print_process(report_prefix: str, *, step: int, eval_info: Optional[Dict[str, Any]] = None, step_duration: Optional[float] = None,
                   start_elapsed: Optional[float] = None, complete_frac: float = -1, num_seqs: int = -1, seq_idx: int = -1,
                   log_memory_usage_device: Optional[str] = None):
    """per-step log line at verbosity 5"""
    if not log.verbose[5]:
        return
    info = [report_prefix, "step %i" % step]
    if eval_info:
        info += ["%s %s" % (k, ("%.3e" % v) if (abs(v) > 1e4 or (0 < abs(v) < 1e-3)) else ("%.3f" % v)) for k, v in eval_info.items()]
    if log_memory_usage_device and log_memory_usage_device.startswith("cuda"):
        info += ["mem_usage:%s %.1fGB" % (log_memory_usage_device, torch.cuda.max_memory_allocated(log_memory_usage_device) / 2 ** 30)]
    if step_duration is not None:
        info += ["%.3f sec/step" % step_duration]
    if start_elapsed is not None:
        info += ["elapsed %s" % hms(start_elapsed)]
    if complete_frac is not None and complete_frac > 0:
        if start_elapsed is not None:
            total = start_elapsed / max(complete_frac, 1e-9)
            info += ["exp. remaining %s" % hms(max(total - start_elapsed, 0))]
        info += ["complete %.02f%%" % (complete_frac * 100)]
    elif num_seqs > 0 and seq_idx >= 0:
        info += ["complete %.02f%%" % (100.0 * (seq_idx + 1) / num_seqs)]
    print(", ".join(info), file=log.v5)
