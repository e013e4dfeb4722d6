"""
Engine base: bookkeeping of model files per epoch, resume rules, cleanup of old checkpoints.

Model files are ``<model>.<epoch:03d>.pt`` (+ ``.opt.pt`` for the optimizer). For training, only epochs whose optimizer
file exists count as resumable. Resume rules (``get_epoch_model``): existing checkpoints of this ``model`` prefix win
over ``load``; ``load`` is used as import when nothing exists (or always for non-train tasks, or with an explicit
``start_epoch``); ``import_model_train_epoch1`` initialises epoch 1; ``start_epoch=1`` forces a fresh start;
``load_epoch`` picks one of the existing epochs.

Parity: returnn/engine/base.py (get_existing_models :75-119, get_epoch_model :135-213, get_train_start_epoch :216-236,
epoch_model_filename :239-249, cleanup_old_models :325-440).
"""

from __future__ import annotations
from typing import Any, Dict, Optional, Set, Tuple
import os
import re
import sys
from ..config import Config
from ..log import log
from ..learning_rate_control import load_learning_rate_control_from_config, LearningRateControl
from ..utils.basic import CollectionReadCheckCovered, human_bytes_size, next_power_of_two

MODEL_POSTFIX = ".pt"
OPT_POSTFIX = ".opt.pt"


def get_checkpoint_filepattern(filepath: str) -> str:
    """strip the .pt / .opt.pt / .meta / .index extension"""
    for ext in (".opt.pt", ".pt", ".safetensors", ".meta", ".index"):
        if filepath.endswith(ext):
            return filepath[: -len(ext)]
    return filepath


def model_epoch_from_filename(filename: str) -> int:
    """``model.042`` -> 42"""
    m = re.match(r".*\.([0-9]+)$", get_checkpoint_filepattern(filename))
    assert m, "cannot get epoch from model filename %r" % filename
    return int(m.group(1))


class EngineBase:
    """base of the torch engine"""

    FORWARD_COMPATIBLE = True

    def __init__(self, config: Optional[Config] = None):
        if config is None:
            from ..config import get_global_config

            config = get_global_config(auto_create=True)
        self.config = config
        self.epoch = 0
        self.global_train_step = 0
        self.model_filename: Optional[str] = None
        self.learning_rate = 0.0
        self.learning_rate_control: Optional[LearningRateControl] = None

    def init_network_from_config(self, config: Optional[Config] = None):
        """load or create the model"""
        raise NotImplementedError

    def init_train_from_config(self, config: Optional[Config] = None):
        """prepare training: LR control etc."""
        if not config:
            config = self.config
        self.learning_rate_control = load_learning_rate_control_from_config(config)
        self.learning_rate = self.learning_rate_control.default_learning_rate

    @classmethod
    def config_get_final_epoch(cls, config: Config) -> int:
        """``num_epochs``, default 5"""
        num_epochs = config.int("num_epochs", 5)
        if config.has("load_epoch"):
            num_epochs = max(num_epochs, config.int("load_epoch", 0))
        return num_epochs

    @classmethod
    def epoch_model_filename(cls, model_filename: str, epoch: int, *, is_pretrain: bool = False) -> str:
        """``<model>[.pretrain].<epoch:03d>``"""
        return model_filename + (".pretrain" if is_pretrain else "") + ".%03d" % epoch

    @classmethod
    def get_existing_models(cls, config: Config, *, for_training: Optional[bool] = None) -> Dict[int, str]:
        """epoch -> model filename without extension"""
        model_filename = config.value("model", "")
        if not model_filename:
            return {}
        if for_training is None:
            for_training = config.value("task", "train") == "train"
        found: Dict[int, str] = {}
        for epoch in range(1, cls.config_get_final_epoch(config) + 1):
            fn = cls.epoch_model_filename(model_filename, epoch)
            if os.path.exists(fn + MODEL_POSTFIX):
                if for_training and not os.path.exists(fn + OPT_POSTFIX):
                    continue
                found[epoch] = fn
        return found

    @classmethod
    def get_start_epoch_no_existing_model(cls, config: Config) -> int:
        """start epoch when nothing exists"""
        mode = config.value("start_epoch", "auto")
        if mode == "auto":
            return 1
        start_epoch = int(mode)
        assert start_epoch >= 1
        return start_epoch

    @classmethod
    def get_epoch_model(cls, config: Config) -> Tuple[Optional[int], Optional[str]]:
        """:return: (epoch of the model to load, its filename without extension)"""
        mode = config.value("start_epoch", "auto")
        start_epoch = None if mode == "auto" else int(mode)
        assert start_epoch is None or start_epoch >= 1
        task = config.value("task", "train")
        load_fn = get_checkpoint_filepattern(config.value("load", ""))
        if load_fn:
            assert os.path.exists(load_fn + MODEL_POSTFIX) or os.path.exists(load_fn), (
                "config option load=%r, file %r does not exist" % (config.value("load", ""), load_fn + MODEL_POSTFIX))
        import_fn = get_checkpoint_filepattern(config.value("import_model_train_epoch1", ""))
        if import_fn:
            assert os.path.exists(import_fn + MODEL_POSTFIX)
        existing = cls.get_existing_models(config)
        load_epoch = config.int("load_epoch", -1)
        if load_fn:
            if load_epoch <= 0:
                try:
                    load_epoch = model_epoch_from_filename(load_fn)
                except AssertionError:
                    load_epoch = 1
        elif load_epoch > 0:
            assert load_epoch in existing, "load_epoch %i: no such model; have %r" % (load_epoch, sorted(existing))
            load_fn = existing[load_epoch]
        if load_fn and (task != "train" or start_epoch is not None):
            epoch_model = (None if (task == "train" and start_epoch is not None) else load_epoch, load_fn)
        elif existing:
            epoch_model = sorted(existing.items())[-1]
            if load_fn:
                print("note: there is a 'load' which we ignore because of existing model", file=log.v4)
        elif task == "train" and import_fn and start_epoch in (None, 1):
            epoch_model = (0, import_fn)
        elif load_fn:
            epoch_model = (load_epoch, load_fn)
        else:
            epoch_model = (None, None)
        if start_epoch == 1:
            if epoch_model[0]:
                print("warning: there is an existing model: %s" % (epoch_model,), file=log.v4)
                epoch_model = (None, None)
        elif (start_epoch or 0) > 1:
            if epoch_model[0]:
                if epoch_model[0] != start_epoch - 1:
                    print("warning: start_epoch %i but there is %s" % (start_epoch, epoch_model), file=log.v4)
                epoch_model = (start_epoch - 1, existing[start_epoch - 1])
        return epoch_model

    @classmethod
    def get_train_start_epoch(cls, config: Config) -> int:
        """the epoch after the last resumable checkpoint"""
        if config.value("start_batch", "auto") != "auto":
            raise Exception("custom start_batch %r not supported" % config.value("start_batch", "auto"))
        last_epoch, _ = cls.get_epoch_model(config)
        return 1 if last_epoch is None else last_epoch + 1

    def get_epoch_model_filename(self, epoch: Optional[int] = None) -> str:
        """filename (without extension) for the epoch"""
        if not epoch:
            epoch = self.epoch
        return self.epoch_model_filename(self.model_filename, epoch)

    def get_epoch_str(self) -> str:
        """for logging"""
        return "epoch %s" % self.epoch

    def _do_save(self) -> bool:
        """only rank 0, not in dry-run"""
        from ..utils.basic import should_write_to_disk

        return should_write_to_disk(config=self.config)

    def delete_model(self, filename: str) -> int:
        """delete all files of one checkpoint. :return: bytes freed"""
        count = 0
        for ext in (MODEL_POSTFIX, OPT_POSTFIX):
            fn = filename + ext
            if os.path.exists(fn):
                count += os.stat(fn).st_size
                os.remove(fn)
        return count

    def cleanup_old_models(self, ask_for_confirmation: bool = False):
        """
        Delete checkpoints except: the last ``keep_last_n`` (2), the ``keep_best_n`` (4) best per score key, and the
        epochs of ``keep`` (default: a sparse pattern growing with the number of epochs).
        """
        if not self._do_save():
            return
        opts = CollectionReadCheckCovered(self.config.get_of_type("cleanup_old_models", dict, {}))
        existing = self.get_existing_models(config=self.config, for_training=False)
        lr_control = self.learning_rate_control or load_learning_rate_control_from_config(self.config)
        epochs = sorted(existing.keys())
        if not epochs:
            print("Cannot cleanup models, no models found.", file=log.v2)
            return
        keep_last_n = opts.get("keep_last_n", 2)
        keep_best_n = opts.get("keep_best_n", 4)
        assert keep_last_n >= 1 and keep_best_n >= 0
        if max(keep_last_n, keep_best_n) >= len(epochs):
            print("Only %i epochs stored so far and keeping last %i epochs and best %i epochs, thus not cleaning up any epochs yet." % (
                len(epochs), keep_last_n, keep_best_n), file=log.v2)
            return
        last = epochs[-1]
        if last <= 10:
            every, doubles = 4, 5
        elif last <= 50:
            every, doubles = 20, 5
        elif last <= 100:
            every, doubles = 40, 10
        else:
            every, doubles = 80 * next_power_of_two(1 + last // 240), 20
        pattern: Set[int] = set(range(every, last + 1, every))
        n = doubles
        while n <= last:
            pattern.add(n)
            n *= 2
        keep: Set[int] = set(opts.get("keep", pattern))
        keep.update(epochs[-keep_last_n:])
        score_values: Dict[str, list] = {}
        for epoch in epochs:
            if epoch in lr_control.epoch_data:
                for k, v in lr_control.epoch_data[epoch].error.items():
                    score_values.setdefault(k, []).append(v)
        for key, scores in sorted(score_values.items()):
            if min(scores) == max(scores):
                print("Ignoring score key %r because all epochs have the same value %r." % (key, scores[0]), file=log.v3)
                continue
            worst = max(scores)
            ranked = sorted((lr_control.epoch_data[e].error.get(key, worst) if e in lr_control.epoch_data else worst, e) for e in epochs)
            keep.update(e for _, e in ranked[:keep_best_n])
        keep.intersection_update(epochs)
        if len(keep) == len(epochs):
            print("%i epochs stored so far and keeping all." % len(epochs), file=log.v2)
            return
        remove = sorted(set(epochs).difference(keep))
        print("We have stored models for epochs %s and keep epochs %s." % (
            epochs if len(epochs) <= 6 else "[%s, ..., %s]" % (", ".join(map(str, epochs[:3])), ", ".join(map(str, epochs[-3:]))),
            sorted(keep)), file=log.v3)
        print("We will delete the models of epochs %s." % (remove,), file=log.v3)
        opts.assert_all_read()
        if self.config.bool("dry_run", False):
            print("Dry-run, will not delete models.", file=log.v2)
            return
        if ask_for_confirmation:
            if input("Delete those models? [y/N] ").strip().lower() not in ("y", "yes"):
                sys.exit(1)
        freed = sum(self.delete_model(existing[e]) for e in remove)
        print("Deleted %s." % human_bytes_size(freed), file=log.v2)

    def _is_dataset_evaluated(self, name: str, *, epoch: Optional[int] = None) -> bool:
        """whether the LR-control database has scores ``<name>_*`` for the epoch"""
        if epoch is None:
            epoch = self.epoch
        if not self.learning_rate_control or epoch not in self.learning_rate_control.epoch_data:
            return False
        return any(k.startswith(name + "_") for k in self.learning_rate_control.epoch_data[epoch].error)
