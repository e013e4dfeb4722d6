"""
Pretraining schedules: a sequence of model constructions that grows over the first epochs.

Two forms are supported:

* **net-dict growing** (the original scheme): given a network description as a dict of layers (``{name: {"class": ...,
  "from": [...]}}``), build step ``i`` with only the first ``i + 1`` hidden layers on the path from input to output
  (``construction_algo`` ``"from_input"`` or ``"from_output"``), or call a custom function
  ``construction_algo(idx, net_dict) -> net_dict | None``. With RF models the dict is whatever ``get_model`` consumes, e.g.
  an encoder description built via ``rf.build_from_dict``.
* **no network modifications**: only the repetitions/epoch mapping is used (``"no_network_modifications"``), e.g. to
  vary ``num_layers`` through ``get_model(epoch=...)`` together with :func:`Pretrain.get_train_num_epochs`.

Parity: returnn/pretrain.py (Pretrain :33-468, pretrain_from_config :471-505).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, List, Optional, Sequence, Union
import copy


class WrapEpochValue:
    """a value of the model description that depends on the pretrain epoch: ``WrapEpochValue(lambda epoch: ...)``"""

    def __init__(self, func):
        self.func = func

    def get_value(self, epoch: int):
        """``func(epoch=epoch)``"""
        return self.func(epoch=epoch)


class Pretrain:
    """list of per-step network dicts + repetitions"""

    def __init__(self, original_network_json: Dict[str, Any], network_init_args=None, copy_param_mode: Optional[str] = None,
                 copy_output_layer: Union[None, bool, str] = None, greedy: Optional[bool] = None, repetitions: Union[None, int, List[int], Dict] = None,
                 construction_algo: Union[str, Callable] = "from_output", output_layers: Sequence[str] = ("output",), input_layers: Sequence[str] = ("data",)):
        """
        :param original_network_json: the full network description
        :param copy_param_mode: None, "ifpossible", "subset", "reset": how parameters move from one step to the next
        :param copy_output_layer: same for the output layer (default: like copy_param_mode, else "ifpossible")
        :param greedy: train only the newest layer and the output
        :param repetitions: epochs per step: int, list (last value repeats), or dict ``{step|"default"|"final": n}``
        :param construction_algo: "from_output", "from_input", "no_network_modifications" or a callable
        """
        assert copy_param_mode in (None, "ifpossible", "subset", "reset")
        if copy_output_layer is None:
            copy_output_layer = copy_param_mode or "ifpossible"
        if copy_output_layer == "reset":
            copy_output_layer = False
        self.copy_param_mode = copy_param_mode
        self.copy_output_layer = copy_output_layer
        self.greedy = bool(greedy)
        self.network_init_args = network_init_args
        self._original = original_network_json
        self._inputs = tuple(input_layers)
        self._outputs = tuple(output_layers)
        self._steps: List[Dict[str, Any]] = []
        if construction_algo == "from_input":
            self._construct(from_input=True)
        elif construction_algo == "from_output":
            self._construct(from_input=False)
        elif construction_algo == "no_network_modifications":
            self._steps = [copy.deepcopy(original_network_json)]
        elif callable(construction_algo):
            self._construct_custom(construction_algo)
        else:
            raise ValueError("invalid construction_algo %r" % (construction_algo,))
        n = len(self._steps)
        if not repetitions:
            repetitions = 1
        if isinstance(repetitions, dict):
            rep = dict(repetitions)
            reps = [rep.pop("default", 1)] * n
            for k, v in sorted(rep.items(), key=lambda kv: str(kv[0])):
                reps[n - 1 if k == "final" else int(k)] = v
        else:
            reps = [repetitions] if isinstance(repetitions, int) else list(repetitions)
            assert 0 < len(reps) <= n
            reps = reps + [reps[-1]] * (n - len(reps))
        for i, net in enumerate(self._steps):
            if "#repetition" in net:
                reps[i] = net.pop("#repetition")
        self.repetitions: List[int] = reps
        self._epoch_to_step: List[int] = [i for i, r in enumerate(reps) for _ in range(r)]

    # -- construction ------------------------------------------------------------------------------------------------
    def _sources(self, layer: Dict[str, Any]) -> List[str]:
        src = layer.get("from", "data")
        if isinstance(src, str):
            src = [src]
        return [s for s in src if isinstance(s, str)]

    def _path_layers(self) -> List[str]:
        """hidden layers on the main path from the output back to the input, in input -> output order"""
        net = self._original
        path: List[str] = []
        cur = [o for o in self._outputs if o in net]
        seen = set(cur)
        while cur:
            nxt = []
            for name in cur:
                for s in self._sources(net[name]):
                    base = s.split("/")[0].lstrip("base:")
                    if base in net and base not in seen and base not in self._inputs:
                        seen.add(base)
                        nxt.append(base)
                        path.append(base)
            cur = nxt
        return list(reversed(path))

    def _subnet(self, keep_hidden: List[str]) -> Dict[str, Any]:
        """the outputs plus the kept hidden layers; a source that was dropped is replaced by the last kept layer before it"""
        net = self._original
        order = self._path_layers()
        keep = set(keep_hidden)
        res: Dict[str, Any] = {}

        def resolve(name: str) -> List[str]:
            if name not in net or name in keep or name in self._inputs:
                return [name]
            out: List[str] = []
            for s in self._sources(net[name]):
                out.extend(resolve(s))
            return out or list(self._inputs)

        for name in list(keep_hidden) + [o for o in self._outputs if o in net]:
            layer = copy.deepcopy(net[name])
            srcs: List[str] = []
            for s in self._sources(layer):
                for r in resolve(s):
                    if r not in srcs:
                        srcs.append(r)
            if "from" in layer or srcs != ["data"]:
                layer["from"] = srcs
            res[name] = layer
        # layers off the main path (e.g. auxiliary losses) whose sources all exist
        for name, layer in net.items():
            if name in res or name in order or not isinstance(layer, dict):
                if name not in res and not isinstance(layer, dict):
                    res[name] = layer  # "#..." meta entries
                continue
            if all(s in res or s in self._inputs for s in self._sources(layer)):
                res[name] = copy.deepcopy(layer)
        return res

    def _construct(self, *, from_input: bool):
        order = self._path_layers()
        if not order:
            self._steps = [copy.deepcopy(self._original)]
            return
        for i in range(1, len(order) + 1):
            keep = order[:i] if from_input else order[-i:]
            self._steps.append(self._subnet(keep))
        self._steps[-1] = copy.deepcopy(self._original)

    def _construct_custom(self, func: Callable):
        idx = 0
        while True:
            net = func(idx, copy.deepcopy(self._original))
            if net is None:
                break
            self._steps.append(net)
            idx += 1
            assert idx < 1000, "construction_algo never returned None"
        self._steps.append(copy.deepcopy(self._original))

    # -- queries -----------------------------------------------------------------------------------------------------
    def get_train_num_epochs(self) -> int:
        """epochs covered by the schedule"""
        return len(self._epoch_to_step)

    def get_final_network_json(self) -> Dict[str, Any]:
        """the full network"""
        return self._steps[-1]

    def get_network_json_for_epoch(self, epoch: int) -> Dict[str, Any]:
        """:param epoch: 1-based; after the schedule: the full network"""
        if epoch > len(self._epoch_to_step):
            return self._steps[-1]
        return self._steps[self._epoch_to_step[epoch - 1]]

    def get_train_param_args_for_epoch(self, epoch: int) -> Optional[Dict[str, Any]]:
        """greedy mode: which layers train in this epoch"""
        if not self.greedy or epoch > len(self._epoch_to_step):
            return None
        step = self._epoch_to_step[epoch - 1]
        if step == 0:
            return None
        prev = set(self._steps[step - 1].keys())
        new = [k for k in self._steps[step].keys() if k not in prev]
        return {"layers": new + list(self._outputs)}

    def __str__(self):
        parts = ["Pretrain construction algo, %i steps, %i epochs:" % (len(self._steps), self.get_train_num_epochs())]
        for i, (net, r) in enumerate(zip(self._steps, self.repetitions)):
            parts.append("  step %i (x%i): %s" % (i, r, sorted(k for k in net.keys() if not k.startswith("#"))))
        return "\n".join(parts)


def pretrain_from_config(config) -> Optional[Pretrain]:
    """
    :param config: reads ``pretrain`` (``"default"`` or a dict of :class:`Pretrain` args) and ``network``
    :return: the schedule or None
    """
    opts = config.typed_value("pretrain", None) or config.value("pretrain", "")
    if not opts:
        return None
    net = config.typed_value("network", None)
    if net is None:
        get_network = config.typed_value("get_network", None)
        assert callable(get_network), "pretrain needs `network` or `get_network` in the config"
        net = get_network(epoch=10 ** 9)
    if opts == "default":
        return Pretrain(original_network_json=net)
    assert isinstance(opts, dict), "pretrain: expected 'default' or a dict, got %r" % (opts,)
    opts = dict(opts)
    if "repetitions" not in opts and config.has("pretrain_repetitions"):
        opts["repetitions"] = config.typed_value("pretrain_repetitions")
    return Pretrain(original_network_json=net, **opts)
