"""
Entry point: ``rnn.py <config> [++key value ...]`` / ``python -m returnn_b200 <config> ...``.

Sequence: ``init_config`` (priority: defaults < config files < command line) -> log -> fault handlers -> backend
(device checks, distributed process group) -> ``startup_callback`` -> datasets -> engine -> ``task``.

Tasks: ``train``, ``eval``, ``forward`` (alias ``search``), ``compute_priors``, ``analyze_data``,
``cleanup_old_models``, ``initialize_model``, ``nop``, ``nop_init_net_train``, ``debug_shell``, ``config:<function>``.

Parity: returnn/__main__.py (init_config :54-129, load_data :169-218, setup_dummy_datasets :221-262, init_engine :282-306,
init_backend_engine :338-476, init :510-550, finalize :553-574, execute_main_task :589-738, analyze_data :742-793,
main :796-816).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Sequence, Tuple
import os
import sys
import time
import numpy

from .config import Config, set_global_config, get_global_config
from .log import log
from .datasets.basic import Dataset, init_dataset, init_dataset_via_str
from .utils.basic import BackendEngine, BehaviorVersion, get_fwd_compat_kwargs

config: Optional[Config] = None
engine = None
train_data: Optional[Dataset] = None
dev_data: Optional[Dataset] = None
eval_data: Optional[Dataset] = None
quit_returnn = False


def init_config(config_filename: Optional[str] = None, command_line_options: Sequence[str] = (), default_config: Optional[Dict[str, Any]] = None,
                extra_updates: Optional[Dict[str, Any]] = None):
    """
    Build the global config.

    :param config_filename: config file (more can follow as leading entries of command_line_options)
    :param command_line_options: ``sys.argv[1:]`` style
    :param default_config: lowest priority
    :param extra_updates: highest priority
    """
    global config
    config = Config()
    config_filenames = []
    if config_filename:
        config_filenames.append(config_filename)
    opts = list(command_line_options)
    while opts and not opts[0].startswith("-") and not opts[0].startswith("+"):
        config_filenames.append(opts.pop(0))
    if default_config:
        config.update(default_config)
    if extra_updates:
        config.update(extra_updates)
    if opts:
        config.parse_cmd_args(opts)
    for fn in config_filenames:
        config.load_file(fn)
    # command line and extra updates override the files
    if opts:
        config.parse_cmd_args(opts)
    if extra_updates:
        config.update(extra_updates)
    set_global_config(config)
    if config.has("behavior_version"):
        BehaviorVersion.set(config.int("behavior_version", 0))
    if not config.has("task"):
        config.set("task", "train")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", config.value("PYTORCH_CUDA_ALLOC_CONF", "") or os.environ.get("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True"))
    if config.bool("patch_atfork", False):
        from .utils.native_helpers import maybe_restart_with_atfork_patch

        maybe_restart_with_atfork_patch()


def init_log():
    """log sinks from the config"""
    log.init_by_config(config)


def get_cache_byte_sizes() -> Tuple[int, int, int]:
    """``cache_size`` split over train / dev / eval"""
    from .utils.basic import parse_human_size

    cache_sizes_user = config.list("cache_size", ["0"])
    sizes = [parse_human_size(s) for s in cache_sizes_user]
    while len(sizes) < 3:
        sizes.append(sizes[-1] // 2 if len(sizes) == 1 else sizes[-1])
    if len(cache_sizes_user) == 1:
        sizes = [int(sizes[0] * 0.5), int(sizes[0] * 0.25), int(sizes[0] * 0.25)]
    return sizes[0], sizes[1], sizes[2]


def load_data(cfg: Config, cache_byte_size: int, files_config_key: str, **kwargs) -> Optional[Dataset]:
    """dataset from config key ``train`` / ``dev`` / ``eval`` (dict, or legacy string)"""
    default_kwargs = dict(kwargs)
    default_kwargs.setdefault("name", files_config_key)
    if cfg.is_typed(files_config_key) and not isinstance(cfg.typed_value(files_config_key), str):
        opts = cfg.typed_value(files_config_key)
        if opts is None:
            return None
        return init_dataset(opts, default_kwargs=default_kwargs)
    s = cfg.value(files_config_key, "")
    if not s:
        return None
    return init_dataset_via_str(config_str=s, config=cfg, cache_byte_size=cache_byte_size, **default_kwargs)


def init_data():
    """train / dev / eval datasets"""
    global train_data, dev_data, eval_data
    if config.bool("use_dummy_datasets", False):
        setup_dummy_datasets()
    train_cache, dev_cache, eval_cache = get_cache_byte_sizes()
    task = config.value("task", "train")
    chunking = config.typed_value("chunking", None) if config.is_typed("chunking") else config.value("chunking", None)
    seq_ordering = config.value("batching", "default")
    dev_data = load_data(config, dev_cache, "dev", seq_ordering="sorted", **({} ))
    eval_data = load_data(config, eval_cache, "eval", seq_ordering="sorted")
    if task in ("train", "nop_init_net_train", "compute_priors") or config.bool("need_data", False):
        train_data = load_data(config, train_cache, "train", seq_ordering=seq_ordering)
    else:
        train_data = None


def setup_dummy_datasets():
    """``use_dummy_datasets``: replace train/dev/eval by random data generated from ``extern_data``"""
    from .torch.data.extern_data import extern_data_template_from_config_opts

    extern_data_dict = config.typed_value("extern_data")
    assert extern_data_dict, "use_dummy_datasets needs extern_data"
    template = {k: v for k, v in extern_data_template_from_config_opts(extern_data_dict).data.items() if k != "seq_tag"}
    num_seqs = config.int("dummy_dataset_num_seqs", 1000)
    opts = config.typed_value("dummy_dataset_opts", None) or {}
    for key in ("train", "dev", "eval"):
        if key == "eval" and not config.has("eval"):
            continue
        n = num_seqs if key == "train" else max(num_seqs // 10, 1)
        config.set(key, {"class": "DummyGenericDataset", "data_template": template, "num_seqs": n, **opts,
                         **({"fixed_random_seed": 1} if key != "train" else {})})


def print_task_properties():
    """dataset summary"""
    if train_data:
        print("Train data:", file=log.v2)
        print("  input:", train_data.num_inputs, "x", train_data.window, file=log.v2)
        print("  output:", train_data.num_outputs, file=log.v2)
        print(" ", train_data.__class__.__name__, train_data.name, file=log.v2)
    if dev_data:
        print("Dev data:", dev_data.__class__.__name__, dev_data.name, file=log.v2)
    if eval_data:
        print("Eval data:", eval_data.__class__.__name__, eval_data.name, file=log.v2)


def init_engine():
    """create the torch engine"""
    global engine
    from .torch.engine import Engine

    engine = Engine(config=config)


def returnn_greeting(config_filename: Optional[str] = None, command_line_options: Optional[Sequence[str]] = None):
    """start banner"""
    from . import __long_version__

    print("returnn_b200 starting up, version %s, date/time %s, pid %i, cwd %s, Python %s" % (
        __long_version__, time.strftime("%Y-%m-%d-%H-%M-%S (UTC%z)"), os.getpid(), os.getcwd(), sys.executable), file=log.v3)
    if config_filename:
        print("config filename: %s" % config_filename, file=log.v4)
    if command_line_options:
        print("command line options: %s" % (list(command_line_options),), file=log.v4)
    from .utils.basic import get_hostname

    print("Hostname:", get_hostname(), file=log.v4)


def init_backend_engine():
    """select torch, run device diagnostics, set up distributed"""
    BackendEngine.select_engine(config=config)
    import torch
    from .torch.util import diagnose_gpu

    print("PyTorch:", torch.__version__, file=log.v3)
    device = config.value("device", None)
    if device in (None, "gpu") or (device and device.startswith("cuda")):
        res = diagnose_gpu.timeout("torch.cuda.is_available()", timeout_sec=config.float("cuda_init_timeout_sec", 60.0)) if config.bool("torch_check_cuda_in_subproc", False) else "skip"
        if res is None:
            print("Warning: the CUDA availability check did not return; continuing", file=log.v2)
    if torch.cuda.is_available() and log.verbose[4]:
        diagnose_gpu.print_available_devices(file=log.v4)
    if config.typed_value("torch_distributed") is not None:
        from .torch import distributed as _dist

        _dist.get_ctx(config=config)
    if config.bool("use_lovely_tensors", False):
        try:
            import lovely_tensors

            lovely_tensors.monkey_patch()
        except ImportError:
            pass
    _warn_foreign_backend_options()


def _warn_foreign_backend_options():
    foreign = [k for k in ("network", "use_tensorflow", "tf_session_opts", "horovod_reduce_type", "jax_distributed") if config.has(k)]
    if foreign:
        print("Warning: config options for other backends are ignored here: %s" % ", ".join(foreign), file=log.v2)


def init_faulthandler(sigusr1_chain: bool = False):
    """Python faulthandler + native signal handler (stack traces on SIGSEGV etc., thread dump on SIGUSR1)"""
    from .utils import debug

    debug.init_faulthandler(sigusr1_chain=sigusr1_chain)


def init(config_filename: Optional[str] = None, command_line_options: Sequence[str] = (), config_updates: Optional[Dict[str, Any]] = None,
         extra_greeting: Optional[str] = None):
    """everything before the task runs"""
    from .utils import better_exchook

    better_exchook.install()
    init_config(config_filename=config_filename, command_line_options=command_line_options, extra_updates=config_updates)
    if config.bool("use_train_proc_manager", False):
        from .utils.train_proc_manager import maybe_start_train_proc_manager

        maybe_start_train_proc_manager(config=config)
    init_log()
    if extra_greeting:
        print(extra_greeting, file=log.v1)
    returnn_greeting(config_filename=config_filename, command_line_options=command_line_options)
    init_faulthandler()
    if config.bool("watch_memory", False):
        from .utils.watch_memory import watch_memory

        watch_memory()
    init_backend_engine()
    if config.bool("use_hot_reloading", False):
        from .utils import hot_reload

        hot_reload.enable(config)
    startup_callback = config.typed_value("startup_callback")
    if startup_callback:
        startup_callback(config=config, **get_fwd_compat_kwargs())
    if need_data():
        init_data()
    print_task_properties()
    init_engine()


def finalize(error_occurred: bool = False):
    """shut down: datasets, process group"""
    global quit_returnn, engine
    print("Quitting", file=getattr(log, "v4", sys.stderr))
    quit_returnn = True
    sys.exited = True
    engine = None
    for ds in (train_data, dev_data, eval_data):
        if ds is not None:
            try:
                ds.finish_epoch(free_resources=True)
            except Exception:
                pass
    import torch.distributed

    if torch.distributed.is_available() and torch.distributed.is_initialized():
        if not error_occurred:
            try:
                torch.distributed.barrier()
            except Exception:
                pass
        torch.distributed.destroy_process_group()
        from .torch import distributed as _dist

        _dist.reset_ctx()


def need_data() -> bool:
    """whether datasets must be loaded for the task"""
    if config.has("need_data") and not config.bool("need_data", True):
        return False
    task = config.value("task", "train")
    if task in ("nop", "nop_init_net_train", "cleanup_old_models", "initialize_model", "debug_shell") or task.startswith("config:"):
        return task == "nop_init_net_train"
    return True


def execute_main_task():
    """run config ``task``"""
    from .utils.basic import BackendEngine

    task = config.value("task", "train")
    if config.is_true("dry_run"):
        print("Dry run, will not save anything.", file=log.v1)
    if task == "train":
        assert train_data is not None, "no train data (config 'train')"
        engine.init_train_from_config(config, train_data, dev_data, eval_data)
        engine.train()
    elif task == "eval":
        epoch = config.int("epoch", -1)
        load_epoch = config.int("load_epoch", -1)
        if epoch >= 0:
            assert load_epoch < 0 or load_epoch == epoch, "epoch and load_epoch have to match"
            config.set("load_epoch", epoch)
        engine.init_train_from_config(config, None, dev_data, eval_data) if config.has("optimizer") else _init_eval_only()
        engine.epoch = max(engine.epoch - 1, 0) if config.value("task", "") == "train" else engine.epoch
        engine.eval_model()
    elif task in ("forward", "search"):
        assert eval_data is not None or config.has("forward_data"), "no eval data (config 'eval' or 'forward_data')"
        engine.init_network_from_config(config)
        dataset = eval_data
        if config.has("forward_data"):
            fd = config.typed_value("forward_data")
            if isinstance(fd, str) and fd in ("train", "dev", "eval"):
                dataset = {"train": train_data, "dev": dev_data, "eval": eval_data}[fd]
            else:
                dataset = init_dataset(fd, default_kwargs={"name": "forward_data"})
        callback = config.typed_value("forward_callback")
        assert callback, "no forward_callback specified"
        if callable(callback) and not hasattr(callback, "process_seq"):
            callback = callback()
        engine.forward_with_callback(dataset=dataset, callback=callback)
    elif task == "compute_priors":
        assert train_data is not None, "train data for priors should be provided"
        engine.init_network_from_config(config)
        from .torch.util.compute_priors import compute_priors

        compute_priors(engine=engine, dataset=train_data, config=config)
    elif task == "analyze":
        data = eval_data or dev_data
        assert data is not None, "task analyze: no 'eval' or 'dev' data"
        engine.init_network_from_config(config)
        engine.analyze(data=data, statistics=config.list("statistics", None))
    elif task == "analyze_data":
        analyze_data(config)
    elif task == "search_server":
        engine.init_network_from_config(config)
        engine.web_server(port=config.int("web_server_port", 12380))
    elif task == "cleanup_old_models":
        engine.cleanup_old_models(ask_for_confirmation=True)
    elif task == "initialize_model":
        engine.init_network_from_config(config)
        engine._updater = None
        engine.epoch = max(engine.epoch, 1) - 1 if engine.epoch else 0
        engine.epoch = 0 if not engine.epoch else engine.epoch
        engine._save_model()
    elif task == "nop":
        print("Task: No-operation", file=log.v1)
    elif task == "nop_init_net_train":
        print("Task: No-operation, despite initializing the network (for training)", file=log.v1)
        engine.init_train_from_config(config, train_data, dev_data, eval_data)
    elif task == "debug_shell":
        from .utils import debug

        debug.debug_shell(user_ns={"config": config, "engine": engine}, user_global_ns=globals())
    elif task.startswith("config:"):
        name = task[len("config:"):]
        func = config.typed_value(name)
        assert callable(func), "task %r: config[%r] is not callable" % (task, name)
        func()
    else:
        raise Exception("unknown task: %r" % (task,))
    print("elapsed: %s" % _hms(time.time() - _start_time), file=log.v3)


def _init_eval_only():
    engine.learning_rate_control = None
    from .learning_rate_control import load_learning_rate_control_from_config

    engine.learning_rate_control = load_learning_rate_control_from_config(config)
    engine.eval_datasets.clear()
    if dev_data:
        engine.eval_datasets["dev"] = dev_data
    if eval_data:
        engine.eval_datasets["eval"] = eval_data
    for name, ds in engine.eval_datasets.items():
        engine._eval_dataloaders[name] = engine._create_data_loader(ds, train=False, dataset_name=name)
    engine.init_network_from_config(config)
    engine._train_step_func = config.typed_value("train_step")


def _hms(s: float) -> str:
    from .utils.basic import hms_fraction

    return hms_fraction(s)


def analyze_data(cfg: Config):
    """mean / std-dev / label priors over the train data; written to ``<statistics_save_prefix>.*``"""
    from .utils.basic import Stats

    ds = train_data
    assert ds is not None
    ds.init_seq_order(epoch=1)
    target = cfg.value("target", "classes")
    stats = Stats()
    n_labels = ds.get_data_dim(target) if target in ds.get_data_keys() else 0
    priors = numpy.zeros((n_labels,), dtype="float64") if n_labels and ds.is_data_sparse(target) else None
    seq_idx = 0
    total_targets = 0
    while ds.is_less_than_num_seqs(seq_idx):
        ds.load_seqs(seq_idx, seq_idx + 1)
        x = ds.get_data(seq_idx, "data")
        if not ds.is_data_sparse("data"):
            stats.collect(x)
        if priors is not None:
            t = ds.get_data(seq_idx, target)
            priors += numpy.bincount(t.reshape(-1), minlength=n_labels)[:n_labels]
            total_targets += t.size
        seq_idx += 1
    stats.dump(output_file_prefix=cfg.value("statistics_save_prefix", None), stream=log.v1)
    if priors is not None and total_targets:
        priors /= total_targets
        print("Label priors:", priors, file=log.v1)
        prefix = cfg.value("statistics_save_prefix", None)
        if prefix:
            numpy.savetxt("%s.priors.txt" % prefix, priors)
            numpy.savetxt("%s.log_priors.txt" % prefix, numpy.log(numpy.maximum(priors, 1e-30)))


_start_time = time.time()


def main(argv: Optional[Sequence[str]] = None):
    """``argv[0]`` is the program name"""
    global _start_time
    if argv is None:
        argv = sys.argv
    _start_time = time.time()
    return_code = 0
    error = False
    try:
        assert len(argv) >= 2, "usage: %s <config>" % argv[0]
        init(command_line_options=argv[1:])
        execute_main_task()
    except KeyboardInterrupt:
        return_code = 1
        error = True
        print("KeyboardInterrupt", file=getattr(log, "v3", sys.stderr))
        if getattr(log, "verbose", [False] * 6)[5]:
            sys.excepthook(*sys.exc_info())
    except BaseException:
        error = True
        finalize(error_occurred=True)
        raise
    finalize(error_occurred=error)
    if return_code:
        sys.exit(return_code)


if __name__ == "__main__":
    main(sys.argv)
