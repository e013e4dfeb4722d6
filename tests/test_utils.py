"""CPU tests of the utility modules: bpe, fsa builders, lru cache, math helpers, pretty printer, numpy backend, pretrain schedules,
hot reload, torch array helpers, inf/nan tracer, native code compiler."""

import io
import itertools
import os
import sys
import time

import numpy
import pytest
import torch


def test_bpe_standard_and_sampling(tmp_path):
    from returnn_b200.utils.bpe import StandardBytePairEncoder, SamplingBytePairEncoder, PrefixTree, BpeOpts, CharSyncSearch

    codes = tmp_path / "codes.txt"
    codes.write_text("#version: 0.2\nl o\nlo w</w>\ne r</w>\nn e\nne w\nnew er</w>\n")
    bpe = StandardBytePairEncoder(str(codes))
    assert bpe.segment_sentence("low newer lower") == ["low", "newer", "lo@@", "w@@", "er"]
    bpe2 = StandardBytePairEncoder(str(codes), labels=["low", "n@@", "e@@", "w@@", "er", "l@@", "o@@", "ne@@"])
    assert bpe2.segment_sentence("newer") == ["ne@@", "w@@", "er"]
    labels = ["a", "b", "ab", "a@@", "b@@", "ab@@", "c"]
    tree = PrefixTree(opts=BpeOpts(label_postfix_merge_symbol="@@"))
    for lab in labels:
        tree.add(lab)
    segs = sorted(CharSyncSearch(tree, "abab").search())
    assert segs == [["a@@", "b@@", "a@@", "b"], ["a@@", "b@@", "ab"], ["ab@@", "a@@", "b"], ["ab@@", "ab"]]
    greedy = SamplingBytePairEncoder(labels=labels, breadth_prob=0.0, rnd=numpy.random.RandomState(1), unknown_label="<unk>")
    assert greedy.segment_sentence("abab abc x") == ["ab@@", "ab", "ab@@", "c", "<unk>"]
    fine = SamplingBytePairEncoder(labels=labels, breadth_prob=1.0, rnd=numpy.random.RandomState(1), unknown_label="<unk>")
    assert fine.segment_sentence("abab") == ["a@@", "b@@", "a@@", "b"]
    for seg in (greedy, fine):
        assert "".join(s.replace("@@", "") for s in seg.segment_sentence("abab")) == "abab"


def test_fsa_ctc_unique_paths_and_builders():
    from returnn_b200.utils import fsa as F

    batch = F.get_ctc_fsa_fast_bw(targets=numpy.array([[1, 2, 2], [3, 0, 0]]), seq_lens=numpy.array([3, 1]), blank_idx=0)
    assert batch.edges.shape[0] == 4 and batch.start_end_states.shape == (2, 2)

    def count_paths(b, string):
        e = batch.edges
        states = {int(batch.start_end_states[0, b]): 1}
        for ch in string:
            nxt = {}
            for i in range(e.shape[1]):
                if e[3, i] == b and e[2, i] == ch and int(e[0, i]) in states:
                    nxt[int(e[1, i])] = nxt.get(int(e[1, i]), 0) + states[int(e[0, i])]
            states = nxt
        return states.get(int(batch.start_end_states[1, b]), 0)

    def collapse(s):
        return [x for x in (k for k, _ in itertools.groupby(s)) if x != 0]

    for s in itertools.product([0, 1, 2], repeat=5):
        assert count_paths(0, s) == (1 if collapse(s) == [1, 2, 2] else 0), s
    g = F.Graph("ab ba")
    F.Ctc(g).run()
    assert g.num_states_ctc == 2 * 5 + 1
    F.Asg(F.Graph("aab")).run()
    hmm = F.Hmm(F.Graph("hi yo"))
    hmm.load_lexicon({"hi": [["h", "i"]], "yo": [["y", "o"], ["j", "o"]]})
    assert hmm.run().num_states_hmm == 3 + 5 + 2 * 5
    stairs = F.fast_bw_fsa_staircase([3, 2], with_loop=True, max_skip=1)
    assert stairs.edges.shape[1] == 13
    shared = F.FastBwFsaShared()
    shared.add_inf_loop(0, 4)
    assert shared.get_fast_bw_fsa(2).edges.shape == (4, 8)


def test_lru_cache_and_math():
    from returnn_b200.utils.lru_cache import lru_cache
    from returnn_b200.utils.math import PiecewiseLinear, StepFunction, next_power_of_two, ceil_div, merge_random_seeds, simplify_and_format_number

    calls = []

    @lru_cache(maxsize=2)
    def f(x):
        calls.append(x)
        return 2 * x

    f(1), f(2), f(3)
    assert f.cache_len() == 2 and f.cache_peek(1) is None and f.cache_peek(3) == 6
    f.cache_set(7, 99)
    assert f(7) == 99 and 7 not in calls
    assert f.cache_pop(7) == 99 and f.cache_peek(7, fallback="no") == "no"
    f.cache_set_maxsize(1)
    assert f.cache_len() == 1
    f.cache_clear()
    assert f.cache_info().currsize == 0
    assert abs(PiecewiseLinear({0: 0.0, 10: 1.0})(5) - 0.5) < 1e-9 and PiecewiseLinear({1: 3.0})(100) == 3.0
    step = StepFunction({0: 1, 5: 2})
    assert step(4) == 1 and step(5) == 2 and step(-3) == 1
    assert next_power_of_two(17) == 32 and next_power_of_two(1) == 1 and ceil_div(7, 2) == 4
    assert merge_random_seeds([1, 2]) != merge_random_seeds([2, 1]) and simplify_and_format_number(3.0) == "3"


def test_pprint_and_collect_outputs():
    from returnn_b200.utils.pprint import pformat
    from returnn_b200.utils.collect_outputs_dict import CollectOutputsDict, is_key_allowed_in_collect_outputs_dict

    obj = {"a": 1, "net": {"x": [1, 2, 3], "y": {"class": "linear", "n_out": 5}}, "t": (1,), "arr": numpy.arange(3)}
    text = pformat(obj)
    back = eval(text, {"numpy": numpy})
    assert back["net"] == obj["net"] and back["t"] == (1,) and list(back["arr"]) == [0, 1, 2]
    d = CollectOutputsDict(allowed_key_patterns=["enc_*", "out"])
    d["enc_3"] = 1
    d["dec_1"] = 2
    d.update({"out": 3, "other": 4})
    assert dict(d) == {"enc_3": 1, "out": 3} and not is_key_allowed_in_collect_outputs_dict(d, "x") and is_key_allowed_in_collect_outputs_dict({}, "x")


def test_numpy_backend():
    from returnn_b200.tensor import Tensor, Dim, batch_dim
    import returnn_b200.frontend as rf

    t = Dim(None, name="t")
    t.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=numpy.array([3, 2], dtype="int32"))
    x = Tensor("x", dims=[batch_dim, t], dtype="float32", raw_tensor=numpy.arange(6, dtype="float32").reshape(2, 3))
    y = x * 2.0 + 1.0
    assert isinstance(y.raw_tensor, numpy.ndarray) and y.raw_tensor.tolist() == [[1.0, 3.0, 5.0], [7.0, 9.0, 11.0]]
    assert (x > 2.0).raw_tensor.tolist() == [[False, False, False], [True, True, True]]
    assert rf.reduce_sum(x, axis=t).raw_tensor.tolist() == [3.0, 7.0]  # the padded frame of the second sequence is ignored
    assert rf.reduce_mean(x, axis=t).raw_tensor.tolist() == [1.0, 3.5]
    assert rf.reduce_max(x, axis=t).raw_tensor.tolist() == [2.0, 4.0]
    # torch tensors are untouched by the dispatch
    a = Tensor("a", dims=[batch_dim], dtype="float32", raw_tensor=torch.ones(2))
    assert isinstance((a + 1).raw_tensor, torch.Tensor)


def test_pretrain_schedule():
    from returnn_b200.pretrain import Pretrain

    net = {"l1": {"class": "linear", "from": "data"}, "l2": {"class": "linear", "from": "l1"}, "l3": {"class": "linear", "from": "l2"},
           "output": {"class": "softmax", "from": "l3"}}
    p = Pretrain(net, repetitions={"default": 2, "final": 1})
    assert p.get_train_num_epochs() == 5
    assert sorted(p.get_network_json_for_epoch(1)) == ["l3", "output"] and p.get_network_json_for_epoch(1)["l3"]["from"] == ["data"]
    assert p.get_network_json_for_epoch(5) == net and p.get_network_json_for_epoch(99) == net
    p2 = Pretrain(net, construction_algo="from_input")
    assert sorted(p2.get_network_json_for_epoch(1)) == ["l1", "output"] and p2.get_network_json_for_epoch(1)["output"]["from"] == ["l1"]
    p3 = Pretrain(net, construction_algo=lambda idx, d: None if idx >= 1 else {"output": dict(d["output"], **{"from": "data"})})
    assert p3.get_train_num_epochs() == 2


def test_hot_reload(tmp_path):
    from returnn_b200.utils.hot_reload import ConfigHotReloader

    mod = tmp_path / "usermod_hot_reload_test.py"
    mod.write_text("def f():\n    return 1\n")
    sys.path.insert(0, str(tmp_path))
    try:
        import usermod_hot_reload_test as m

        cfg = {"train_step": m.f, "nested": {"fns": [m.f]}, "n": 3}
        reloader = ConfigHotReloader(cfg)
        assert reloader.modules == ["usermod_hot_reload_test"] and not reloader.any_module_changed()
        mod.write_text("def f():\n    return 2\n")
        future = time.time() + 5
        os.utime(str(mod), (future, future))
        assert reloader.any_module_changed()
        reloader.reload_changed_modules()
        assert cfg["train_step"]() == 2 and cfg["nested"]["fns"][0]() == 2 and cfg["n"] == 3
    finally:
        sys.path.remove(str(tmp_path))
        sys.modules.pop("usermod_hot_reload_test", None)


def test_torch_array_helpers_and_tracer():
    from returnn_b200.torch.util import array_, scaled_gradient, rope, module as module_util
    from returnn_b200.torch.util.debug_inf_nan import debug_inf_nan

    x = torch.arange(24.0).reshape(2, 3, 4).requires_grad_(True)
    m = torch.tensor([[1, 0, 1], [0, 1, 1]], dtype=torch.bool)
    out, n = array_.masked_select_bound(x, m, bound=5)
    assert out.shape == (5, 4) and int(n) == 4 and torch.equal(out[:4], x[m]) and float(out[4].abs().sum()) == 0.0
    out.sum().backward()
    assert torch.equal(x.grad[:, :, 0], m.float())
    assert torch.equal(array_.masked_select(x, m), x[m]) and array_.nonzero(m.flatten(), out_len=4).tolist() == [0, 2, 4, 5]
    assert array_.sequence_mask(torch.tensor([1, 3])).tolist() == [[True, False, False], [True, True, True]]
    assert array_.sequence_mask_time_major(torch.tensor([1, 3])).shape == (3, 2)
    y = torch.ones(3, requires_grad=True)
    scaled_gradient.scaled_gradient(y, -2.0).sum().backward()
    assert y.grad.tolist() == [-2.0, -2.0, -2.0]
    ang = torch.rand(5, 4)
    v = torch.randn(5, 8)
    r = rope.apply_rope(v, torch.cat([ang.sin(), ang.cos()], -1))
    torch.testing.assert_close(r.norm(dim=-1), v.norm(dim=-1))  # a rotation
    lin = torch.nn.Linear(2, 2)
    module_util.convert_parameters_to_buffers(lin, ["bias"], persistent=False)
    assert "bias" not in dict(lin.named_parameters()) and "bias" not in lin.state_dict() and lin(torch.zeros(1, 2)).shape == (1, 2)
    buf = io.StringIO()
    debug_inf_nan(lambda: torch.log(torch.zeros(3)) * 0, file=buf, report_every_op_call=False)
    assert "aten::log" in buf.getvalue() and "3 inf" in buf.getvalue()


def test_native_code_compiler(tmp_path, monkeypatch):
    from returnn_b200.utils import basic
    from returnn_b200.utils.native_code_compiler import NativeCodeCompiler

    monkeypatch.setattr(basic, "get_cache_dir", lambda: str(tmp_path))
    src = 'extern "C" int add(int a, int b) { return a + b; }'
    c = NativeCodeCompiler("t_add", code=src)
    assert c.load_lib_ctypes().add(2, 3) == 5
    mtime = os.path.getmtime(c.get_lib_filename())
    c2 = NativeCodeCompiler("t_add", code=src)
    assert c2.get_lib_filename() == c.get_lib_filename() and os.path.getmtime(c2.get_lib_filename()) == mtime  # cached
    with pytest.raises(RuntimeError):
        NativeCodeCompiler("t_bad", code="this is not C++")


def test_rf_native_dim_helpers():
    """the CPython extension gives the same answers as the Python specification"""
    from returnn_b200.frontend import _native
    from returnn_b200.tensor import Dim, Tensor, batch_dim

    mod = _native.get_module()
    if mod is None:
        pytest.skip("extension not built")
    a, b, c = Dim(3, name="a"), Dim(4, name="b"), Dim(None, name="c")
    assert mod.match_dims((a, b, c), (c, a, b)) == [2, 0, 1] and mod.match_dims((a, b), (c, a)) == [-1, 0]
    assert mod.match_dims((a, a), (a, a)) == [0, 1]  # a repeated dim is matched once per occurrence
    assert mod.same_dims((a, b), (a, b)) and not mod.same_dims((a, b), (b, a)) and not mod.same_dims((a,), (a, b))
    assert mod.merge_dims((a, b), (b,)) == (a, b) and mod.merge_dims((b,), (a, b)) == (a, b)
    assert mod.merge_dims((a,), (b,)) == (a, b) and mod.merge_dims((), (b,)) == (b,) and mod.merge_dims((a, c), (c, b)) == (a, c, b)
    x = Tensor("x", dims=[batch_dim, a, b], dtype="float32", raw_tensor=torch.zeros(2, 3, 4))
    assert x.get_out_permutation_to_dims([b, batch_dim, a]) == [2, 0, 1]
    with pytest.raises(ValueError):
        x.get_out_permutation_to_dims([b, batch_dim, c])
    y = Tensor("y", dims=[b], dtype="float32", raw_tensor=torch.ones(4))
    assert (x + y).dims == (batch_dim, a, b) and (y + x).dims == (batch_dim, a, b)
    # raw views: permutation, size-1 axes for missing dims, the identical tensor when nothing changes
    raw = torch.arange(24.0).reshape(2, 3, 4)
    assert mod.copy_compatible_raw(raw, (batch_dim, a, b), (batch_dim, a, b)) is raw
    v = mod.copy_compatible_raw(raw, (batch_dim, a, b), (b, c, batch_dim, a))
    assert tuple(v.shape) == (4, 1, 2, 3) and torch.equal(v[:, 0], raw.permute(2, 0, 1)) and v.data_ptr() == raw.data_ptr()
    with pytest.raises(ValueError):
        mod.copy_compatible_raw(raw, (batch_dim, a, b), (a, b))
    # operand preparation of a binary op: same dims tuple, scalar, subset, disjoint dims
    dims = (batch_dim, a, b)
    ra, rb, out = mod.bin_op_prepare(raw, dims, raw, dims)
    assert ra is raw and rb is raw and out is dims
    ra, rb, out = mod.bin_op_prepare(raw, dims, torch.tensor(2.0), ())
    assert ra is raw and out == dims and rb.ndim == 0
    ra, rb, out = mod.bin_op_prepare(torch.ones(4), (b,), raw, dims)
    assert out == dims and tuple(ra.shape) == (1, 1, 4) and rb is raw
    ra, rb, out = mod.bin_op_prepare(torch.ones(3), (a,), torch.ones(5), (c,))
    assert out == (a, c) and tuple(ra.shape) == (3, 1) and tuple(rb.shape) == (1, 5)
    # through the frontend: the results equal plain torch broadcasting
    import returnn_b200.frontend as rf

    z = Tensor("z", dims=[b, batch_dim], dtype="float32", raw_tensor=torch.arange(8.0).reshape(4, 2))
    xr = Tensor("x", dims=[batch_dim, a, b], dtype="float32", raw_tensor=raw)
    s = xr * z
    assert s.dims == (batch_dim, a, b) and torch.equal(s.raw_tensor, raw * torch.arange(8.0).reshape(4, 2).t()[:, None, :])
    assert torch.equal((xr > 11.0).raw_tensor, raw > 11.0) and torch.equal(rf.maximum(xr, 5.0).raw_tensor, raw.clamp_min(5.0))
    assert torch.equal(xr.copy_compatible_to_dims_raw([a, b, batch_dim]), raw.permute(1, 2, 0))


def test_tools_on_small_inputs(tmp_path):
    """command line tools that need no trained model: Bliss readers, word/symbol collection, pickle dump, file cache"""
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    corpus = tmp_path / "corpus.xml"
    corpus.write_text('<?xml version="1.0" encoding="utf8"?>\n<corpus name="c"><recording name="r1" audio="/nonexistent/r1.wav">'
                      '<segment name="s1" start="0.0" end="1.5"><orth> hello world </orth></segment>'
                      '<segment name="s2" start="1.5" end="4.0"><orth>foo bar hello</orth></segment></recording></corpus>\n')

    def run(tool, *args):
        proc = subprocess.run([sys.executable, os.path.join(root, "tools", tool)] + [str(a) for a in args], stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=120)
        assert proc.returncode == 0, proc.stderr.decode()[-2000:]
        return proc.stdout.decode()

    assert eval(run("bliss-collect-seq-lens.py", corpus)) == {"c/r1/s1": 150, "c/r1/s2": 250}
    assert run("bliss-dump-text.py", corpus, "--with-names").splitlines() == ["c/r1/s1 hello world", "c/r1/s2 foo bar hello"]
    assert run("bliss-get-segment-names.py", corpus).split() == ["c/r1/s1", "c/r1/s2"]
    assert run("collect-words.py", corpus).splitlines()[0] == "hello 2"
    assert "'h' 2" in run("collect-orth-symbols.py", corpus)
    run("bliss-to-ogg-zip.py", corpus, "--output", tmp_path / "c.zip", "--no-audio")
    import zipfile

    with zipfile.ZipFile(str(tmp_path / "c.zip")) as zf:
        entries = eval(zf.read("c.txt").decode())
    assert [e["seq_name"] for e in entries] == ["c/r1/s1", "c/r1/s2"] and entries[1]["text"] == "foo bar hello"
    import pickle

    (tmp_path / "x.pkl").write_bytes(pickle.dumps({"a": [1, 2]}))
    assert eval(run("dump-pickle.py", tmp_path / "x.pkl")) == {"a": [1, 2]}


def test_task_system_pickler_sends_config_functions_by_value(tmp_path):
    """functions, classes, closures and recursion from an exec'd module survive a trip into a fresh interpreter; big arrays use shared memory"""
    import subprocess
    import sys
    import os
    import numpy
    from returnn_b200.utils import task_system as ts

    src = (
        "import numpy\nSCALE = 3\n"
        "def helper(x):\n    return x * SCALE\n"
        "def fn(x, *, k=2):\n    return helper(x) + k + int(numpy.sum([1, 2]))\n"
        "def fact(n):\n    return 1 if n <= 1 else n * fact(n - 1)\n"
        "class Aug:\n    factor = 5\n    def __init__(self, a):\n        self.a = a\n    def __call__(self, x):\n        return helper(x) * self.factor + self.a\n"
        "def make_closure(c):\n    def inner(x):\n        return x + c\n    return inner\n")
    g = {"__name__": "__returnn_config__"}
    exec(compile(src, "cfg", "exec"), g)
    objs = {"fn": g["fn"], "fact": g["fact"], "aug": g["Aug"](7), "clo": g["make_closure"](11), "lam": (lambda x: x * 2),
            "arr": numpy.arange(600000, dtype="float32"), "mod": numpy, "meth": g["Aug"](1).__call__}
    fn = tmp_path / "objs.pkl"
    fn.write_bytes(ts.dumps(objs, shared_mem=True))
    assert fn.stat().st_size < 10000  # the 2.4 MB array went through shared memory
    code = ("import pickle; o = pickle.load(open(%r, 'rb')); "
            "print(o['fn'](4), o['fact'](5), o['aug'](2), o['clo'](1), o['lam'](21), int(o['arr'][-1]), o['mod'].__name__, o['meth'](1))" % str(fn))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.check_output([sys.executable, "-c", code], cwd=root, env=dict(os.environ, PYTHONPATH=root)).decode().split()
    assert out == ["17", "120", "37", "12", "42", "599999", "numpy", "16"]
    # importable functions still go by name
    assert b"numpy" in ts.dumps(numpy.sum) and len(ts.dumps(numpy.sum)) < 100
    sh = ts.SharedNumpyArray.from_array(numpy.arange(10))
    sh2 = ts.loads(ts.dumps(sh))
    sh2.array[3] = 77
    assert sh.array[3] == 77
    sh2.close()
    sh.close()
    assert ts.next_power_of_two(5) == 8 and ts.next_power_of_two(8) == 8


def test_fsa_store_and_command_line(tmp_path, capsys):
    from returnn_b200.utils import fsa as F

    g = F.main(["--fsa", "ctc", "--label_seq", "ab", "--file", "ctc_ab", "--path", str(tmp_path), "--file_format", "dot"])
    out = capsys.readouterr().out
    assert "ctc automaton of 'ab': 5 states" in out and g.num_states_ctc == 5
    dot = (tmp_path / "ctc_ab.dot").read_text()
    assert dot.startswith("digraph fsa {") and '0 -> 1 [label="a"]' in dot and "4 [shape=doublecircle]" in dot and dot.count("->") == len(g.edges_ctc)
    g2 = F.main(["--fsa", "asg", "--label_seq", "aab", "--label_conversion", "--single_state"])
    assert g2.num_states_asg > 0
    st = F.Store(2, [F.Edge(0, 1, 97, 0.5)])
    assert 'label="a(97) / 0.5"' in st.fsa_to_dot_format()


def test_better_exchook_statement_names_chain_and_threads():
    import io
    import sys
    from returnn_b200.utils import better_exchook as B

    def inner(alpha, table):
        beta = {"k": [1, 2, 3]}
        return (alpha +
                table["missing"] +
                len(beta))

    def outer():
        try:
            inner(41, {"present": 1})
        except KeyError as exc:
            raise ValueError("outer failed") from exc

    buf = io.StringIO()
    try:
        outer()
    except ValueError:
        B.better_exchook(*sys.exc_info(), file=buf, with_color=False, autodebugshell=False)
    text = buf.getvalue()
    # both exceptions of the chain, oldest first, joined by the standard sentence
    assert text.index("KeyError: 'missing'") < text.index("direct cause") < text.index("ValueError: outer failed")
    # the whole three-line statement and the values of the names in it
    assert "return (alpha +" in text and 'table["missing"] +' in text and "len(beta))" in text
    assert "alpha = <local> 41" in text and "table = <local> {'present': 1}" in text and "beta = <local> {'k': [1, 2, 3]}" in text
    assert "len = " not in text  # builtins are not listed
    src, first = B.get_source_statement(__file__, inner.__code__.co_firstlineno + 3)
    assert src.startswith("return (alpha +") and src.endswith("len(beta))") and first == inner.__code__.co_firstlineno + 2
    assert list(B.iter_names_in_source("f(a.b.c, key=x) + y.z")) == ["f", "a", "a.b", "a.b.c", "x", "y", "y.z"]
    col = B.Color(True)
    assert col("x", "red", bold=True) == "\x1b[1;31mx\x1b[0m" and B.Color(False)("x", "red") == "x"
    out = io.StringIO()
    B.dump_all_thread_tracebacks(file=out)
    assert "MainThread" in out.getvalue() and "dump_all_thread_tracebacks" in out.getvalue()
    lines = B.format_tb(sys._getframe(), limit=1, with_color=False)
    assert any("test_better_exchook_statement_names_chain_and_threads" in ln for ln in lines)


def test_basic_helpers(tmp_path, capsys):
    import io
    import sys
    from returnn_b200.utils import basic as U

    assert U.model_epoch_from_filename("net/model.042.pt") == 42 and U.model_epoch_from_filename("m.pretrain.007") == 7
    assert U.get_checkpoint_filepattern("a/b.010.pt") == "a/b.010" and U.get_checkpoint_filepattern("a/b.010.opt.pt") == "a/b.010" and U.get_model_filename_postfix() == ".pt"
    assert U.find_ranges([1, 2, 3, 7, 8, 10]) == [(1, 4), (7, 9), (10, 11)]
    assert U.dict_joined({"a": 1}, {"a": 2, "b": 3}) == {"a": 2, "b": 3} and U.dict_zip(["x", "y"], [1, 2]) == {"x": 1, "y": 2}
    assert U.sorted_values_from_dict({"b": 2, "a": 1}) == [1, 2]
    assert U.obj_diff_str({"a": [1, 2]}, {"a": [1, 2]}) == "No diff."
    diff = U.obj_diff_list({"a": [1, 2], "b": 1}, {"a": [1, 3], "c": 1})
    assert any("[1]" in d and "2 != other: 3" in d for d in diff) and any("'b' not in other" in d for d in diff) and any("'c' not in self" in d for d in diff)
    assert U.uniq_generic([[1], [2], [1], numpy.array([1, 2]), numpy.array([1, 2])])[:2] == [[1], [2]] and len(U.uniq_generic([[1], [1]])) == 1
    fd = U.FrozenDict({"a": [1, 2]}) if False else U.make_hashable({"a": [1, {"b": {3, 4}}], "z": numpy.arange(3)})
    assert hash(fd) == hash(U.make_hashable({"a": [1, {"b": {4, 3}}], "z": numpy.arange(3)}))
    with pytest.raises(TypeError):
        fd["x"] = 1
    a, b = [1], [1]
    refs = U.DictRefKeys()
    refs[a] = "a"
    assert a in refs and b not in refs and refs[a] == "a" and len(refs) == 1 and U.RefIdEq(a) != U.RefIdEq(b)
    assert U.ObjAsDict(refs)["_d"] is refs._d and U.DictAsObj({"q": 5}).q == 5
    assert U.attr_chain(sys, ["version_info", "major"]) == 3 and U.camel_case_to_snake_case("HelloWorldHTTPServer") == "hello_world_http_server"
    assert U.str_is_number("1e-3") and not U.str_is_number("x1") and U.unicode_to_str(b"ab") == "ab" and U.prod([2, 3, 4]) == 24 and U.prod([]) == 1
    x = numpy.arange(10).reshape(5, 2)
    assert U.slice_pad_zeros(x, -2, 2).tolist() == [[0, 0], [0, 0], [0, 1], [2, 3]] and U.slice_pad_zeros(x, 4, 7).tolist() == [[8, 9], [0, 0], [0, 0]]
    q = U.random_orthogonal((4, 6), seed=1)
    numpy.testing.assert_allclose(q @ q.T, numpy.eye(4), atol=1e-5)
    acc = numpy.zeros(3)
    U.inplace_increment(acc, numpy.array([0, 0, 2]), numpy.array([1.0, 2.0, 5.0]))
    assert acc.tolist() == [3.0, 0.0, 5.0]
    numpy.testing.assert_allclose(U.softmax(numpy.array([[0.0, 0.0], [1000.0, 0.0]]), axis=1), [[0.5, 0.5], [1.0, 0.0]], atol=1e-9)
    assert U.parse_orthography_into_symbols("hi  [laugh] you") == ["h", "i", " ", "[LAUGH]", " ", "y", "o", "u"]
    assert U.parse_orthography_into_symbols("a b [x]", word_based=True) == ["a", "b", "[X]"]
    assert U.parse_orthography("(a) b", postfix=["[END]"]) == ["a", " ", "b", "[END]"]
    assert U.json_remove_comments('{"a": "x//y", // c\n /* block */ "b": 2}') == '{"a": "x//y",\n  "b": 2}'

    class Base:
        def __init__(self, base_arg, base_opt=1):
            pass

    class Child(Base):
        def __init__(self, child_arg, *, child_kw=2, **kwargs):
            super().__init__(**kwargs)

    assert U.collect_class_init_kwargs(Child) == ["child_arg", "child_kw", "base_arg", "base_opt"]
    assert U.collect_class_init_kwargs(Child, only_with_default=True) == ["child_kw", "base_opt"]
    assert U.collect_mandatory_class_init_kwargs(Child) == ["child_arg", "base_arg"]
    U.help_on_type_error_wrong_args(Child, ["child_arg", "bogus"])
    err = capsys.readouterr().err
    assert "bogus" in err and "base_arg" in err
    assert U.type_attrib_mro_chain(Child, "__init__")[:2] == [Child.__dict__["__init__"], Base.__dict__["__init__"]]
    assert U.next_type_attrib_in_mro_chain(Child, "__init__", Child.__dict__["__init__"]) is Base.__dict__["__init__"]
    assert U.getargspec(Base.__init__).args == ["self", "base_arg", "base_opt"]
    assert U.AsyncThreadRun("t", lambda: 7).get() == 7 and U.wrap_async_func(lambda: 8) == 8
    with pytest.raises(ZeroDivisionError):
        U.AsyncThreadRun("t", lambda: 1 / 0).get()
    with U.guard_infinite_recursion("f", 1):
        with pytest.raises(U.InfiniteRecursionDetected):
            with U.guard_infinite_recursion("f", 1):
                pass
    assert U.try_get_caller_name(depth=0) == "test_basic_helpers"
    f = tmp_path / "sub" / "touched"
    U.maybe_make_dirs(str(tmp_path / "sub"))
    U.touch_file(str(f))
    assert f.exists() and U.is_valid_fd(0) and not U.is_valid_fd(9999)
    (tmp_path / "vec.txt").write_text("1.5\n2\n\n")
    assert U.load_txt_vector(str(tmp_path / "vec.txt")) == [1.5, 2.0]
    buf = io.BytesIO()
    U.write_pickled_object(buf, {"k": [1, 2]})
    buf.seek(0)
    import struct

    (n,) = struct.unpack("<i", buf.read(4))
    assert U.deserialize_object(U.read_bytes_to_new_buffer(buf, n).read()) == {"k": [1, 2]}
    assert U.eval_shell_str("echo 'a b' $HOME")[:2] == ["echo", "a b"] and U.eval_shell_str(lambda: ["x", "$NOPE_NOT_SET"]) == ["x", ""]
    assert U.sys_exec_out("echo", "hi").strip() == "hi" and U.sys_exec_ret_code("false") == 1 and U.sys_cmd_out_lines("printf 'a\\nb\\n'") == ["a", "b"]
    assert U.which("sh") and U.is_64bit_platform() and U.get_number_available_cpus() >= 1 and U.available_physical_memory_in_bytes() > 0
    assert isinstance(U.describe_returnn_version(), str) and "(" in U.describe_torch_version() and U.make_dll_name("x") == "libx.so"
    assert U.escape_c_str('a"b\n') == '"a\\"b\\n"' and U.terminal_size(io.StringIO()) == (-1, -1) and not U.is_tty(io.StringIO())
    assert "cut at 2 items" in U.pretty_print(list(range(10)), limit=2) and U.pretty_print({"a": 1}) == "{'a': 1}"
    U.log_runtime_info_to_dir(str(tmp_path / "logs"))
    assert len(list((tmp_path / "logs").iterdir())) == 1
    from returnn_b200.utils.h5_shim import get_h5py

    with get_h5py().File(str(tmp_path / "t.hdf"), "w") as h:
        h.attrs["numLabels"] = 7
        h.create_dataset("inputs", data=numpy.zeros((5, 3)))
        U.hdf5_strings(h, "labels", ["a", "bcd"])
    assert U.hdf5_dimension(str(tmp_path / "t.hdf"), "numLabels") == 7 and U.hdf5_dimension(str(tmp_path / "t.hdf"), "inputs") == 5
    assert U.hdf5_shape(str(tmp_path / "t.hdf"), "inputs") == (5, 3)


def test_small_named_helpers_of_updater_debug_and_diagnosis(capsys):
    import signal
    import torch
    import returnn_b200.frontend as rf
    from returnn_b200.torch.updater import wrap_user_blacklist_wd_modules
    from returnn_b200.torch.util.distributed import all_reduce_sum
    from returnn_b200.torch.util.diagnose_gpu import print_relevant_env_vars
    from returnn_b200.utils import debug as D

    assert torch.nn.LayerNorm in wrap_user_blacklist_wd_modules(None) and rf.LayerNorm in wrap_user_blacklist_wd_modules(None)
    assert wrap_user_blacklist_wd_modules(["rf.Embedding", "torch.nn.Conv1d", rf.BatchNorm]) == (rf.Embedding, torch.nn.Conv1d, rf.BatchNorm)
    with pytest.raises(AssertionError):
        wrap_user_blacklist_wd_modules(["builtins.dict"])
    x = torch.ones(3, requires_grad=True)
    y = all_reduce_sum(x)
    y.sum().backward()
    assert y.tolist() == [1.0, 1.0, 1.0] and x.grad.tolist() == [1.0, 1.0, 1.0]
    print_relevant_env_vars()
    assert capsys.readouterr().out
    assert D.format_signum(int(signal.SIGSEGV)) == "%i (SIGSEGV)" % int(signal.SIGSEGV)
    old = signal.getsignal(signal.SIGUSR2)
    try:
        signal.signal(signal.SIGUSR2, signal.SIG_DFL)
        assert D.install_signal_handler_if_default(signal.SIGUSR2) and signal.getsignal(signal.SIGUSR2) is D.signal_handler
        assert not D.install_signal_handler_if_default(signal.SIGUSR2)
    finally:
        signal.signal(signal.SIGUSR2, old)
