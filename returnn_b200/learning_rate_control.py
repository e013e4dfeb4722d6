"""
Learning rate control: per-epoch learning rate schedule driven by a score database, persisted as text.

Schedulers: ``constant``, ``newbob`` / ``newbob_rel`` (decay when the relative improvement is below a threshold),
``newbob_abs`` (absolute difference), ``newbob_multi_epoch`` (mean relative improvement over the last N epochs, for
use with ``partition_epoch``). An explicit ``learning_rates`` list (or dict epoch -> lr) overrides the first epochs
(warm-up).

File format (``learning_rate_file``): a Python dict literal ``{epoch: EpochData(learningRate=..., error={...}), ...}``;
meta information is stored inside ``error`` under ``":meta:<key>"``.

Parity: returnn/learning_rate_control.py (LearningRateControl :16-536, NewbobRelative :564-613, NewbobAbs,
NewbobMultiEpoch, load_learning_rate_control_from_config :758-782, save/load :511-536).
"""

from __future__ import annotations
from typing import Any, Dict, List, Optional, Tuple, Union
import os
import numpy
from .log import log
from .utils.basic import better_repr

__all__ = ["LearningRateControl", "ConstantLearningRate", "NewbobRelative", "NewbobAbs", "NewbobMultiEpoch",
           "learning_rate_control_type", "load_learning_rate_control_from_config"]


class LearningRateControl:
    """base class and score database"""

    need_error_info = True

    class EpochData:
        """learning rate, scores/errors and meta info of one epoch"""

        def __init__(self, *, learning_rate: Optional[float] = None, error=None, meta: Optional[Dict[str, Any]] = None, **kwargs):
            if learning_rate is None:
                learning_rate = kwargs.pop("learningRate", None)
            if kwargs:
                raise TypeError("EpochData: unexpected kwargs: %r" % (kwargs,))
            if learning_rate is not None and not isinstance(learning_rate, float):
                if isinstance(learning_rate, int):
                    learning_rate = float(learning_rate)
                else:
                    raise TypeError("EpochData: unexpected learning_rate type: %r" % type(learning_rate))
            self.learning_rate = learning_rate
            if isinstance(error, float):
                error = {"old_format_score": error}
            elif error is None:
                error = {}
            if not isinstance(error, dict):
                raise TypeError("EpochData: unexpected error type: %r" % type(error))
            if meta is None:
                meta = {k[len(":meta:"):]: v for k, v in error.items() if k.startswith(":meta:")}
                error = {k: v for k, v in error.items() if not k.startswith(":meta:")}
            self.error: Dict[str, float] = error
            self.meta: Dict[str, Any] = meta

        def __repr__(self):
            merged = dict(self.error)
            merged.update({":meta:%s" % k: v for k, v in self.meta.items()})
            return "EpochData(learningRate=%s, error=%s)" % (better_repr(self.learning_rate), better_repr(merged))

    @classmethod
    def load_initial_kwargs_from_config(cls, config) -> Dict[str, Any]:
        """constructor kwargs from config keys"""
        return {
            "default_learning_rate": config.float("learning_rate", 1.0),
            "min_learning_rate": config.float("min_learning_rate", 0.0),
            "default_learning_rates": config.typed_value("learning_rates") or config.float_list("learning_rates"),
            "error_measure_key": config.typed_value("learning_rate_control_error_measure") or config.value("learning_rate_control_error_measure", None),
            "relative_error_also_relative_to_learning_rate": config.bool("learning_rate_control_relative_error_relative_lr", False),
            "min_num_epochs_per_new_learning_rate": config.int("learning_rate_control_min_num_epochs_per_new_lr", 0),
            "relative_error_div_by_old": config.bool("newbob_relative_error_div_by_old", False),
            "learning_rate_decay": config.typed_value("learning_rate_decay", config.opt_typed_value("newbob_learning_rate_decay", 0.5)),
            "learning_rate_growth": config.typed_value("learning_rate_growth", config.opt_typed_value("newbob_learning_rate_growth", 1.0)),
            "filename": config.value("learning_rate_file", None),
        }

    @classmethod
    def load_initial_from_config(cls, config) -> "LearningRateControl":
        """instance from config"""
        return cls(**cls.load_initial_kwargs_from_config(config))

    def __init__(self, default_learning_rate: float, min_learning_rate: float = 0.0, default_learning_rates=None,
                 error_measure_key=None, relative_error_also_relative_to_learning_rate: bool = False,
                 min_num_epochs_per_new_learning_rate: int = 0, relative_error_div_by_old: bool = False,
                 learning_rate_decay=1.0, learning_rate_growth=1.0, filename: Optional[str] = None):
        self.epoch_data: Dict[int, LearningRateControl.EpochData] = {}
        self.default_learning_rate = float(default_learning_rate)
        self.min_learning_rate = min_learning_rate
        if default_learning_rates:
            if isinstance(default_learning_rates, str):
                default_learning_rates = eval(default_learning_rates)
            if isinstance(default_learning_rates, (list, tuple)):
                default_learning_rates = {i + 1: v for i, v in enumerate(default_learning_rates)}
            assert isinstance(default_learning_rates, dict)
            for epoch, v in default_learning_rates.items():
                self.set_default_learning_rate_for_epoch(epoch, float(v))
        self.default_learning_rates = default_learning_rates
        self.error_measure_key = error_measure_key
        self.relative_error_also_relative_to_learning_rate = relative_error_also_relative_to_learning_rate
        self.min_num_epochs_per_new_learning_rate = min_num_epochs_per_new_learning_rate
        self.relative_error_div_by_old = relative_error_div_by_old
        self.learning_rate_decay = float(learning_rate_decay) if isinstance(learning_rate_decay, str) else learning_rate_decay
        self.learning_rate_growth = float(learning_rate_growth) if isinstance(learning_rate_growth, str) else learning_rate_growth
        self.filename = filename
        if filename:
            if os.path.exists(filename):
                print("Learning-rate-control: loading file %s" % filename, file=log.v4)
                self.load()
            else:
                print("Learning-rate-control: file %s does not exist yet" % filename, file=log.v4)
        else:
            print("Learning-rate-control: no file specified, not saving history (no proper restart possible)", file=log.v4)

    __repr__ = lambda self: "%s(default_learning_rate=%r, filename=%r)" % (self.__class__.__name__, self.default_learning_rate, self.filename)

    def __str__(self):
        return "%r, epoch data: %s, error key: %s" % (
            self, ", ".join("%i: %s" % (e, d) for e, d in sorted(self.epoch_data.items())), self.get_error_key(epoch=1))

    @staticmethod
    def _apply_update(learning_rate: float, update) -> float:
        if callable(update):
            return float(update(learning_rate))
        return learning_rate * update

    def calc_learning_rate_decay_or_grow(self, learning_rate: float, decay: bool, grow: Optional[bool] = None) -> float:
        """decay (clipped at min_learning_rate) or grow"""
        if grow is None:
            grow = not decay
        assert not (grow and decay)
        if decay:
            learning_rate = max(self._apply_update(learning_rate, self.learning_rate_decay), self.min_learning_rate)
        if grow:
            learning_rate = self._apply_update(learning_rate, self.learning_rate_growth)
        return learning_rate

    def calc_learning_rate_for_epoch(self, epoch: int) -> float:
        """the scheduler rule"""
        raise NotImplementedError

    def _last_epochs_for_epoch(self, epoch: int, num_epochs: int) -> List[int]:
        return sorted(e for e in self.epoch_data if e < epoch)[-num_epochs:] if num_epochs else []

    def calc_new_learning_rate_for_epoch(self, epoch: int) -> float:
        """scheduler rule, but keep a learning rate for at least min_num_epochs_per_new_learning_rate epochs"""
        n = self.min_num_epochs_per_new_learning_rate
        if n > 1:
            last_lrs = [self.epoch_data[e].learning_rate for e in self._last_epochs_for_epoch(epoch, n)]
            if len(set(last_lrs)) >= 2 or 0 < len(last_lrs) < n:
                return last_lrs[-1]
        return self.calc_learning_rate_for_epoch(epoch)

    def get_learning_rate_for_epoch(self, epoch: int) -> float:
        """stored or newly computed (and then stored) learning rate"""
        assert epoch >= 1
        if epoch in self.epoch_data and self.epoch_data[epoch].learning_rate is not None:
            return self.epoch_data[epoch].learning_rate
        lr = self.calc_new_learning_rate_for_epoch(epoch)
        self.set_default_learning_rate_for_epoch(epoch, lr)
        return lr

    def set_default_learning_rate_for_epoch(self, epoch: int, learning_rate: float):
        """store if not yet set"""
        if epoch in self.epoch_data:
            if not self.epoch_data[epoch].learning_rate:
                self.epoch_data[epoch].learning_rate = learning_rate
        else:
            self.epoch_data[epoch] = self.EpochData(learning_rate=float(learning_rate))

    def get_last_epoch(self, epoch: int) -> Optional[int]:
        """last epoch < epoch with data"""
        prev = [e for e in self.epoch_data if e < epoch]
        return max(prev) if prev else None

    def get_most_recent_learning_rate(self, epoch: int, exclude_current: bool = True) -> float:
        """latest known lr up to epoch"""
        for e in sorted(self.epoch_data, reverse=True):
            if e > epoch or (exclude_current and e == epoch):
                continue
            if self.epoch_data[e].learning_rate is None:
                continue
            return self.epoch_data[e].learning_rate
        return self.default_learning_rate

    def calc_relative_error(self, old_epoch: int, new_epoch: int) -> Optional[float]:
        """(new - old) / |new| (or / |old|), optionally rescaled by lr / default lr"""
        old_key, old_error = self.get_epoch_error_key_value(old_epoch)
        new_key, new_error = self.get_epoch_error_key_value(new_epoch)
        if old_error is None or new_error is None or old_key != new_key:
            return None
        denom = abs(old_error) if self.relative_error_div_by_old else abs(new_error)
        rel = (new_error - old_error) / denom
        if self.relative_error_also_relative_to_learning_rate:
            lr = self.get_most_recent_learning_rate(new_epoch, exclude_current=False)
            if lr > 0:
                rel /= lr / self.default_learning_rate
        return rel

    def set_epoch_error(self, epoch: int, error: Dict[str, Union[float, Dict[str, float]]]):
        """add scores of an epoch; nested dicts are flattened as ``<outer>_<inner>``"""
        if epoch not in self.epoch_data:
            print("Learning rate not set for epoch %i. Assuming default." % epoch, file=log.v4)
            self.get_learning_rate_for_epoch(epoch)
        flat: Dict[str, float] = {}
        for k, v in error.items():
            if isinstance(v, dict):
                if len(v) == 1:
                    flat[k] = list(v.values())[0]
                else:
                    for k1, v1 in v.items():
                        if ":" in k1:
                            k1 = k1[k1.index(":") + 1:]
                        flat[k + "_" + k1] = v1
            else:
                flat[k] = v
        for v in flat.values():
            assert isinstance(v, float), "set_epoch_error: scores must be float, got %r" % (flat,)
        self.epoch_data[epoch].error.update(flat)
        if epoch == 1:
            print("Learning-rate-control: error key %r from %r" % (self.get_error_key(epoch), flat), file=log.v4)

    def get_error_key(self, epoch: int) -> Optional[str]:
        """which score drives the schedule: configured key, else dev_score, else any dev_*, else train_score"""
        if epoch not in self.epoch_data:
            if isinstance(self.error_measure_key, list):
                return self.error_measure_key[0]
            return self.error_measure_key
        err = self.epoch_data[epoch].error
        if not err:
            return None
        if len(err) == 1 and "old_format_score" in err:
            return "old_format_score"
        cands: List[str] = []
        wanted = self.error_measure_key if isinstance(self.error_measure_key, list) else ([self.error_measure_key] if self.error_measure_key else [])
        for k in wanted:
            cands += [k, k + "_output"]
        cands += ["dev_score", "dev_score_output"]
        for k in cands:
            if k in err:
                return k
        for pred in (lambda k: k == "dev_score_output/output" or k.startswith("dev_score_output/output_"),
                     lambda k: k.startswith("dev_score_output/"), lambda k: k.startswith("dev_")):
            for k in sorted(err):
                if pred(k):
                    return k
        for k in ("train_score", "train_score_output"):
            if k in err:
                return k
        return min(err.keys())

    def get_epoch_error_dict(self, epoch: int) -> Dict[str, float]:
        """all scores of the epoch"""
        return self.epoch_data[epoch].error if epoch in self.epoch_data else {}

    def get_epoch_error_key_value(self, epoch: int) -> Tuple[Optional[str], Optional[float]]:
        """(key, value) of the driving score"""
        err = self.get_epoch_error_dict(epoch)
        if not err:
            return None, None
        key = self.get_error_key(epoch)
        assert key and key in err, "%r not in %r. fix %r in config. set it to %r or so." % (
            key, err, "learning_rate_control_error_measure", "dev_error")
        return key, err[key]

    def get_epoch_error_value(self, epoch: int) -> Optional[float]:
        """value of the driving score"""
        return self.get_epoch_error_key_value(epoch)[1]

    def get_last_best_epoch(self, last_epoch: int, first_epoch: int = 1, only_last_epochs: Optional[int] = None,
                            filter_score: float = float("inf"), only_last_n: int = -1, min_score_dist: float = 0.0) -> Optional[int]:
        """the epoch in [first_epoch, last_epoch] with the lowest driving score (same key as the latest)"""
        if only_last_epochs:
            first_epoch = max(first_epoch, last_epoch - only_last_epochs + 1)
        if first_epoch > last_epoch:
            return None
        values = [(self.get_epoch_error_key_value(ep), ep) for ep in range(first_epoch, last_epoch + 1)]
        values = [((k, v), ep) for (k, v), ep in values if v is not None]
        if not values:
            return None
        last_key, latest_score = values[-1][0]
        values = [(v, ep) for (k, v), ep in values if k == last_key]
        values = [(v, ep) for v, ep in values if v <= filter_score]
        if not values:
            return None
        if only_last_n >= 1:
            values = values[-only_last_n:]
        values = [(v, ep) for v, ep in values if v + min_score_dist < latest_score or ep == values[-1][1]]
        if len(values) > 1 and min_score_dist > 0:
            values = values[:-1] if any(v + min_score_dist < latest_score for v, _ in values[:-1]) else values
        return min(values)[1] if values else None

    def save(self):
        """write the database (tmp file + rename)"""
        if not self.filename:
            return
        directory = os.path.dirname(self.filename)
        if directory:
            os.makedirs(directory, exist_ok=True)
        tmp = self.filename + ".new_tmp"
        with open(tmp, "w") as f:
            f.write(better_repr(self.epoch_data))
            f.write("\n")
        os.replace(tmp, self.filename)

    def load(self):
        """read the database"""
        s = open(self.filename).read()
        self.epoch_data = eval(s, {"nan": float("nan"), "inf": float("inf"), "EpochData": LearningRateControl.EpochData,
                                   "numpy": numpy, "np": numpy})


class ConstantLearningRate(LearningRateControl):
    """always the default learning rate (or the most recent explicit one)"""

    need_error_info = False

    def calc_learning_rate_for_epoch(self, epoch: int) -> float:
        while epoch > 1:
            epoch -= 1
            if epoch in self.epoch_data and self.epoch_data[epoch].learning_rate is not None:
                return self.epoch_data[epoch].learning_rate
        return self.default_learning_rate


class NewbobRelative(LearningRateControl):
    """decay when the relative error change (new-old)/|new| is above ``newbob_relative_error_threshold`` (default -0.01)"""

    @classmethod
    def load_initial_kwargs_from_config(cls, config):
        kwargs = super().load_initial_kwargs_from_config(config)
        kwargs["relative_error_threshold"] = config.float("newbob_relative_error_threshold", -0.01)
        return kwargs

    def __init__(self, relative_error_threshold: float, **kwargs):
        super().__init__(**kwargs)
        self.relative_error_threshold = relative_error_threshold

    def calc_learning_rate_for_epoch(self, epoch: int) -> float:
        last = self.get_last_epoch(epoch)
        if last is None:
            return self.default_learning_rate
        lr = self.epoch_data[last].learning_rate
        if lr is None:
            return self.default_learning_rate
        last2 = self.get_last_epoch(last)
        if last2 is None:
            return lr
        rel = self.calc_relative_error(last2, last)
        if rel is None:
            return lr
        return self.calc_learning_rate_decay_or_grow(lr, decay=rel > self.relative_error_threshold)


class NewbobAbs(LearningRateControl):
    """decay when new - old is above ``newbob_error_threshold`` (default -0.01)"""

    @classmethod
    def load_initial_kwargs_from_config(cls, config):
        kwargs = super().load_initial_kwargs_from_config(config)
        kwargs["error_threshold"] = config.float("newbob_error_threshold", -0.01)
        return kwargs

    def __init__(self, error_threshold: float, **kwargs):
        super().__init__(**kwargs)
        self.error_threshold = error_threshold

    def calc_learning_rate_for_epoch(self, epoch: int) -> float:
        last = self.get_last_epoch(epoch)
        if last is None:
            return self.default_learning_rate
        lr = self.epoch_data[last].learning_rate
        if lr is None:
            return self.default_learning_rate
        last2 = self.get_last_epoch(last)
        if last2 is None:
            return lr
        old_key, old_error = self.get_epoch_error_key_value(last2)
        new_key, new_error = self.get_epoch_error_key_value(last)
        if old_error is None or new_error is None or old_key != new_key:
            return lr
        return self.calc_learning_rate_decay_or_grow(lr, decay=(new_error - old_error) > self.error_threshold)


class NewbobMultiEpoch(LearningRateControl):
    """mean relative error change over the last ``newbob_multi_num_epochs`` epochs, checked every ``newbob_multi_update_interval``"""

    @classmethod
    def load_initial_kwargs_from_config(cls, config):
        kwargs = super().load_initial_kwargs_from_config(config)
        kwargs.update({
            "num_epochs": config.int("newbob_multi_num_epochs", 5),
            "update_interval": config.int("newbob_multi_update_interval", config.int("newbob_multi_num_epochs", 5)),
            "relative_error_threshold": config.float("newbob_relative_error_threshold", -0.01),
            "relative_error_grow_threshold": config.float("newbob_relative_error_grow_threshold", config.float("newbob_relative_error_threshold", -0.01)),
        })
        return kwargs

    def __init__(self, num_epochs: int, update_interval: int, relative_error_threshold: float, relative_error_grow_threshold: float, **kwargs):
        super().__init__(**kwargs)
        assert num_epochs >= 1 and update_interval >= 1
        self.num_epochs = num_epochs
        self.update_interval = update_interval
        self.relative_error_threshold = relative_error_threshold
        self.relative_error_grow_threshold = relative_error_grow_threshold

    def _calc_recent_mean_relative_error(self, epoch: int) -> Optional[float]:
        epochs = self._last_epochs_for_epoch(epoch, num_epochs=self.num_epochs + 1)
        if len(epochs) <= 1:
            return None
        errs = [self.calc_relative_error(epochs[i], epochs[i + 1]) for i in range(len(epochs) - 1)]
        if any(e is None for e in errs):
            return None
        return float(numpy.mean(errs))

    def calc_learning_rate_for_epoch(self, epoch: int) -> float:
        lr = self.get_most_recent_learning_rate(epoch)
        if self.update_interval > 1 and epoch % self.update_interval != 1:
            return lr
        mean_rel = self._calc_recent_mean_relative_error(epoch)
        if mean_rel is None:
            return lr
        return self.calc_learning_rate_decay_or_grow(lr, decay=mean_rel > self.relative_error_threshold,
                                                     grow=mean_rel < self.relative_error_grow_threshold)


def learning_rate_control_type(type_name: str):
    """class by name"""
    if type_name == "constant":
        return ConstantLearningRate
    if type_name in ("newbob", "newbob_rel", "newbob_relative"):
        return NewbobRelative
    if type_name == "newbob_abs":
        return NewbobAbs
    if type_name == "newbob_multi_epoch":
        return NewbobMultiEpoch
    raise ValueError("unknown learning-rate-control type %r" % type_name)


def load_learning_rate_control_from_config(config) -> LearningRateControl:
    """config ``learning_rate_control`` (default "constant")"""
    control_type = config.value("learning_rate_control", "constant")
    cls = learning_rate_control_type(control_type)
    return cls.load_initial_from_config(config)
