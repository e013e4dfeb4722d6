"""Config (three file formats, command-line overrides, typed access) and Log (reference: returnn/config.py, returnn/log.py)"""

import json
import os
import tempfile
from returnn_b200.config import Config, get_global_config, set_global_config


def test_python_config_typed_values_and_cmdline():
    with tempfile.TemporaryDirectory() as d:
        fn = os.path.join(d, "a.config")
        with open(fn, "w") as f:
            f.write("#!rnn.py\nbatch_size = 5000\nlearning_rate = 0.5\nopt = {'class': 'adam'}\n\ndef get_model(**kw):\n  return 42\n")
        c = Config()
        c.load_file(fn)
        assert c.int("batch_size", 0) == 5000
        assert c.float("learning_rate", 0.0) == 0.5
        assert c.typed_value("opt") == {"class": "adam"}
        assert callable(c.typed_value("get_model")) and c.typed_value("get_model")() == 42
        assert c.is_typed("opt") and c.has("batch_size") and not c.has("nope")
        c.parse_cmd_args(["++batch_size", "123", "++new_key", "abc", "++flag", "True"])
        assert c.int("batch_size", 0) == 123
        assert c.value("new_key", None) == "abc"
        assert c.bool("flag", False) is True


def test_json_and_line_configs():
    with tempfile.TemporaryDirectory() as d:
        fn = os.path.join(d, "b.config")
        with open(fn, "w") as f:
            json.dump({"num_epochs": 3, "task": "train", "lrs": [1, 2]}, f)
        c = Config()
        c.load_file(fn)
        assert c.int("num_epochs", 0) == 3 and c.value("task", "") == "train"
        fn2 = os.path.join(d, "c.config")
        with open(fn2, "w") as f:
            f.write("num_epochs 7\n# comment\nhidden 10,20\n")
        c2 = Config()
        c2.load_file(fn2)
        assert c2.int("num_epochs", 0) == 7
        assert c2.int_list("hidden", []) == [10, 20]


def test_defaults_update_and_global():
    c = Config({"a": 1})
    assert c.int("a", 0) == 1 and c.int("b", 9) == 9
    c.set("b", 2)
    c.update({"c": "x"})
    assert c.int("b", 0) == 2 and c.value("c", "") == "x"
    assert c.bool_or_other("a", None) in (True, 1)
    set_global_config(c)
    assert get_global_config() is c


def test_log_verbosity_streams(capsys):
    from returnn_b200.log import log

    log.initialize(verbosity=[3], logs=[], formatter=[])
    print("shown", file=log.v3)
    print("hidden", file=log.v5)
    out = capsys.readouterr().out
    assert "shown" in out and "hidden" not in out
