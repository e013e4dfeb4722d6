"""
Functional ops of the frontend against the installed reference package (same code run with both, see ``tests/_parity.py``), and
the API additions that need no reference: AMP policy, static-traceable flag, parameter copy behaviour, step-based seeds.
Reference: returnn/frontend/{array_,math_,reduce,attention,label_smoothing,loss,conv,amp,static_traceable}.py.
"""

import numpy
import pytest
import torch

import _parity as P

needs_ref = pytest.mark.skipif(not P.reference_available(), reason="reference package not installed under baseline/_ref")

LENS = [9, 6, 3]


def _inputs(api: P.Api, seed=5):
    """x [B,T,F] float, y [B,T,F] float, idx [B,T] sparse over F, z [B,F2]"""
    rng = numpy.random.RandomState(seed)
    t = api.time_dim(LENS)
    f, f2 = api.Dim(6, name="feat"), api.Dim(4, name="other")
    xv = rng.standard_normal((3, 9, 6)).astype("float32")
    yv = rng.standard_normal((3, 9, 6)).astype("float32")
    iv = rng.randint(0, 6, size=(3, 9)).astype("int32")
    zv = rng.standard_normal((3, 4)).astype("float32")
    return dict(t=t, f=f, f2=f2, x=api.tensor("x", [api.batch_dim, t, f], xv), y=api.tensor("y", [api.batch_dim, t, f], yv),
                idx=api.tensor("idx", [api.batch_dim, t], iv, sparse_dim=f), z=api.tensor("z", [api.batch_dim, f2], zv))


def _np(api, out, order):
    return P.to_numpy_bt(api, out, order)


FUNCS = {
    # name: (function(api, d) -> Tensor, dims order getter, mask?)
    "softmax": lambda api, d: (api.rf.softmax(d["x"], axis=d["f"]), [api.batch_dim, d["t"], d["f"]], True),
    "log_softmax": lambda api, d: (api.rf.log_softmax(d["x"], axis=d["f"]), [api.batch_dim, d["t"], d["f"]], True),
    "softmax_over_time": lambda api, d: (api.rf.softmax(d["x"], axis=d["t"]), [api.batch_dim, d["t"], d["f"]], True),
    "reduce_sum_time": lambda api, d: (api.rf.reduce_sum(d["x"], axis=d["t"]), [api.batch_dim, d["f"]], False),
    "reduce_mean_time": lambda api, d: (api.rf.reduce_mean(d["x"], axis=d["t"]), [api.batch_dim, d["f"]], False),
    "reduce_max_time": lambda api, d: (api.rf.reduce_max(d["x"], axis=d["t"]), [api.batch_dim, d["f"]], False),
    "reduce_logsumexp_feat": lambda api, d: (api.rf.reduce_logsumexp(d["x"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "reduce_argmax_feat": lambda api, d: (api.rf.reduce_argmax(d["x"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "gather": lambda api, d: (api.rf.gather(d["x"], indices=d["idx"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "one_hot": lambda api, d: (api.rf.one_hot(d["idx"]), [api.batch_dim, d["t"], d["f"]], True),
    "combine_add_bc": lambda api, d: (d["x"] + api.rf.reduce_mean(d["y"], axis=d["f"]), [api.batch_dim, d["t"], d["f"]], True),
    "combine_mul": lambda api, d: (d["x"] * d["y"], [api.batch_dim, d["t"], d["f"]], True),
    "compare_where": lambda api, d: (api.rf.where(d["x"] > d["y"], d["x"], d["y"]), [api.batch_dim, d["t"], d["f"]], True),
    "log_add_exp": lambda api, d: (api.rf.log_add_exp(d["x"], d["y"]), [api.batch_dim, d["t"], d["f"]], True),
    "maximum_scalar": lambda api, d: (api.rf.maximum(d["x"], 0.25), [api.batch_dim, d["t"], d["f"]], True),
    "gelu": lambda api, d: (api.rf.gelu(d["x"]), [api.batch_dim, d["t"], d["f"]], True),
    "swish": lambda api, d: (api.rf.swish(d["x"]), [api.batch_dim, d["t"], d["f"]], True),
    "relu_square": lambda api, d: (api.rf.relu_square(d["x"]), [api.batch_dim, d["t"], d["f"]], True),
    "log_sigmoid": lambda api, d: (api.rf.log_sigmoid(d["x"]), [api.batch_dim, d["t"], d["f"]], True),
    "cumsum_time": lambda api, d: (api.rf.cumsum(d["x"], spatial_dim=d["t"]), [api.batch_dim, d["t"], d["f"]], True),
    "reverse_sequence": lambda api, d: (api.rf.reverse_sequence(d["x"], axis=d["t"]), [api.batch_dim, d["t"], d["f"]], True),
    "shift_right": lambda api, d: (api.rf.shift_right(d["x"], axis=d["t"], pad_value=0.0), [api.batch_dim, d["t"], d["f"]], True),
    "matmul_feat": lambda api, d: (api.rf.matmul(d["x"], d["y"], reduce=d["f"]), [api.batch_dim, d["t"]], True),
    "dot_feat_bc": lambda api, d: (api.rf.dot(d["x"], api.rf.reduce_mean(d["y"], axis=d["t"]), reduce=d["f"]), [api.batch_dim, d["t"]], True),
    "sinusoidal_pos": lambda api, d: (api.rf.sinusoidal_positional_encoding(spatial_dim=d["t"], feat_dim=d["f"]), [d["t"], d["f"]], False),
    "label_smoothing": lambda api, d: (api.rf.label_smoothing(d["idx"], 0.1), [api.batch_dim, d["t"], d["f"]], True),
    "cross_entropy": lambda api, d: (api.rf.cross_entropy(estimated=d["x"], estimated_type="logits", target=d["idx"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "smoothed_grad_ce": lambda api, d: (api.rf.cross_entropy(
        estimated=api.rf.label_smoothed_log_prob_gradient(api.rf.log_softmax(d["x"], axis=d["f"]), 0.1, axis=d["f"]), estimated_type="log-probs",
        target=d["idx"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "squared_difference": lambda api, d: (api.rf.squared_difference(d["x"], d["y"]), [api.batch_dim, d["t"], d["f"]], True),
    "clip_by_value": lambda api, d: (api.rf.clip_by_value(d["x"], -0.5, 0.5), [api.batch_dim, d["t"], d["f"]], True),
    "floor_divide_int": lambda api, d: (d["idx"] // 2, [api.batch_dim, d["t"]], True),
    "cast_and_neg": lambda api, d: (-api.rf.cast(d["idx"], "float32"), [api.batch_dim, d["t"]], True),
    "layer_norm_func": lambda api, d: ((d["x"] - api.rf.reduce_mean(d["x"], axis=d["f"])) * api.rf.rsqrt(api.rf.reduce_mean(api.rf.square(d["x"]), axis=d["f"]) + 1e-6),
                                       [api.batch_dim, d["t"], d["f"]], True),
    "moments": lambda api, d: (api.rf.moments(d["x"], axis=[api.batch_dim, d["t"]])[1], [d["f"]], False),
    "range_over_dim": lambda api, d: (api.rf.range_over_dim(d["t"]), [d["t"]], False),
    "sequence_mask": lambda api, d: (api.rf.cast(api.rf.sequence_mask([api.batch_dim, d["t"]]), "float32"), [api.batch_dim, d["t"]], False),
    "top_k_values": lambda api, d: (api.rf.top_k(d["x"], axis=d["f"], k_dim=api.Dim(2, name="k"))[0], None, True),
    "sort_values": lambda api, d: (api.rf.sort(d["x"], axis=d["f"])[0], None, True),
    "expand_dim_and_sum": lambda api, d: (api.rf.reduce_sum(api.rf.expand_dim(d["z"], d["t"]), axis=d["f2"]), [api.batch_dim, d["t"]], True),
    # -- second batch -------------------------------------------------------------------------------------------------------------
    "tanh_sigmoid": lambda api, d: (api.rf.tanh(d["x"]) * api.rf.sigmoid(d["y"]), [api.batch_dim, d["t"], d["f"]], True),
    "exp_log_abs": lambda api, d: (api.rf.log(api.rf.abs(d["x"]) + 1.0) + api.rf.exp(-api.rf.abs(d["y"])), [api.batch_dim, d["t"], d["f"]], True),
    "sqrt_square": lambda api, d: (api.rf.sqrt(api.rf.square(d["x"]) + 1e-3), [api.batch_dim, d["t"], d["f"]], True),
    "minimum_tensor": lambda api, d: (api.rf.minimum(d["x"], d["y"]), [api.batch_dim, d["t"], d["f"]], True),
    "relu_elu_silu": lambda api, d: (api.rf.relu(d["x"]) + api.rf.elu(d["y"]) + api.rf.silu(d["x"]), [api.batch_dim, d["t"], d["f"]], True),
    "reduce_min_feat": lambda api, d: (api.rf.reduce_min(d["x"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "reduce_argmin_feat": lambda api, d: (api.rf.reduce_argmin(d["x"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "reduce_sum_two_axes": lambda api, d: (api.rf.reduce_sum(d["x"], axis=[d["t"], d["f"]]), [api.batch_dim], False),
    "reduce_mean_batch_time": lambda api, d: (api.rf.reduce_mean(d["x"], axis=[api.batch_dim, d["t"]]), [d["f"]], False),
    "reduce_max_time_masked": lambda api, d: (api.rf.reduce_max(d["x"], axis=d["t"], use_mask=True), [api.batch_dim, d["f"]], False),
    "reduce_logsumexp_time": lambda api, d: (api.rf.reduce_logsumexp(d["x"], axis=d["t"]), [api.batch_dim, d["f"]], False),
    "reduce_any_all": lambda api, d: (api.rf.cast(api.rf.reduce_any(d["x"] > 1.0, axis=d["f"]), "float32") + 2.0 * api.rf.cast(
        api.rf.reduce_all(d["x"] > -2.0, axis=d["f"]), "float32"), [api.batch_dim, d["t"]], True),
    "logical_ops": lambda api, d: (api.rf.cast(api.rf.logical_and(d["x"] > 0.0, api.rf.logical_not(d["y"] > 0.0)), "float32"),
                                   [api.batch_dim, d["t"], d["f"]], True),
    "compare_eq_idx": lambda api, d: (api.rf.cast(api.rf.compare(d["idx"], "==", 3), "float32"), [api.batch_dim, d["t"]], True),
    "where_scalar": lambda api, d: (api.rf.where(d["x"] > 0.0, d["x"], 0.5), [api.batch_dim, d["t"], d["f"]], True),
    "concat_feat": lambda api, d: (api.rf.concat((d["x"], d["f"]), (d["y"], d["f"]))[0], None, True),
    "split_feat": lambda api, d: (api.rf.split(d["x"], axis=d["f"], out_dims=[api.Dim(2, name="a"), api.Dim(4, name="b")])[1], None, True),
    "stack_two": lambda api, d: (lambda r: (r[0], list(r[0].dims), False))(api.rf.stack([d["x"], d["y"]], out_dim=api.Dim(2, name="stack"))),
    "merge_split_dims": lambda api, d: (api.rf.split_dims(d["x"], axis=d["f"], dims=[api.Dim(2, name="a"), api.Dim(3, name="b")]), None, True),
    "pad_feat": lambda api, d: (api.rf.pad(d["x"], axes=[d["f"]], padding=[(1, 2)], value=0.5)[0], None, True),
    "slice_feat": lambda api, d: (api.rf.slice(d["x"], axis=d["f"], start=1, end=5)[0], None, True),
    "shift_right_idx": lambda api, d: (api.rf.shift_right(d["idx"], axis=d["t"], pad_value=0), [api.batch_dim, d["t"]], True),
    "cumsum_feat": lambda api, d: (api.rf.cumsum(d["x"], spatial_dim=d["f"]), [api.batch_dim, d["t"], d["f"]], True),
    "gather_time_first": lambda api, d: (api.rf.gather(d["x"], indices=0, axis=d["t"]), [api.batch_dim, d["f"]], False),
    "masked_fill_via_where": lambda api, d: (api.rf.where(api.rf.sequence_mask([api.batch_dim, d["t"]]), d["x"], -1.0), [api.batch_dim, d["t"], d["f"]], False),
    "num_elements_mean": lambda api, d: (api.rf.reduce_sum(d["x"], axis=[api.batch_dim, d["t"]]) / float(sum(LENS)), [d["f"]], False),
    "relative_positional_encoding": lambda api, d: (lambda r: (r[0], [r[1], d["f"]], False))(api.rf.relative_positional_encoding(
        query_spatial_dim=d["t"], key_value_spatial_dim=d["t"], feat_dim=d["f"])),
    "one_hot_times_x": lambda api, d: (api.rf.reduce_sum(api.rf.one_hot(d["idx"]) * d["x"], axis=d["f"]), [api.batch_dim, d["t"]], True),
    "matmul_outer": lambda api, d: (api.rf.matmul(d["x"], d["z"], reduce=[]), None, True),
    "ctc_greedy_like_argmax_shift": lambda api, d: (api.rf.cast(api.rf.reduce_argmax(d["x"], axis=d["f"]) != api.rf.shift_right(
        api.rf.reduce_argmax(d["x"], axis=d["f"]), axis=d["t"], pad_value=-1), "float32"), [api.batch_dim, d["t"]], True),
    "power_and_div": lambda api, d: ((api.rf.abs(d["x"]) + 1.0) ** 1.5 / (api.rf.abs(d["y"]) + 2.0), [api.batch_dim, d["t"], d["f"]], True),
    "floor_ceil_round": lambda api, d: (api.rf.floor(d["x"]) + 2.0 * api.rf.ceil(d["y"]) + 4.0 * api.rf.round(d["x"] * 3.0), [api.batch_dim, d["t"], d["f"]], True),
    "clip_by_value_int": lambda api, d: (api.rf.clip_by_value(d["idx"], 1, 4), [api.batch_dim, d["t"]], True),
    "log_softmax_two_step": lambda api, d: (d["x"] - api.rf.reduce_logsumexp(d["x"], axis=d["f"]), [api.batch_dim, d["t"], d["f"]], True),
    "cosine_similarity_func": lambda api, d: (api.rf.matmul(d["x"], d["y"], reduce=d["f"]) * api.rf.rsqrt(
        api.rf.reduce_sum(api.rf.square(d["x"]), axis=d["f"]) * api.rf.reduce_sum(api.rf.square(d["y"]), axis=d["f"]) + 1e-6), [api.batch_dim, d["t"]], True),
    "kl_div_probs": lambda api, d: (api.rf.reduce_sum(api.rf.softmax(d["x"], axis=d["f"]) * (api.rf.log_softmax(d["x"], axis=d["f"])
                                                                                              - api.rf.log_softmax(d["y"], axis=d["f"])), axis=d["f"]),
                                    [api.batch_dim, d["t"]], True),
}


def _run_func(api, name):
    api.setup()
    d = _inputs(api)
    out, order, do_mask = FUNCS[name](api, d)
    if order is None:
        order = [api.batch_dim, d["t"]] + [x for x in out.dims if x not in (api.batch_dim, d["t"])]
    arr = _np(api, out, order)
    if do_mask and len(order) >= 2 and order[0] == api.batch_dim and order[1] == d["t"]:
        arr = P.masked(arr, LENS)
    return arr


@needs_ref
@pytest.mark.parametrize("name", sorted(FUNCS))
def test_function_equals_reference(name):
    ref = _run_func(P.reference(), name)
    our = _run_func(P.ours(), name)
    P.assert_close(our, ref, atol=2e-6, rtol=1e-5, what=name)


# ---- API additions checked on their own ---------------------------------------------------------------------------------------

def test_unstack_and_stack_roundtrip():
    api = P.ours()
    api.setup()
    rf = api.rf
    d = _inputs(api)
    parts = rf.unstack(d["z"], axis=d["f2"])
    assert len(parts) == 4 and all(p.dims == (api.batch_dim,) for p in parts)
    back, _ = rf.stack(parts, out_dim=d["f2"])
    assert torch.equal(back.copy_transpose([api.batch_dim, d["f2"]]).raw_tensor, d["z"].raw_tensor)
    with pytest.raises(ValueError):
        rf.unstack(d["x"], axis=d["t"])


def test_scatter_count_and_pad_packed():
    api = P.ours()
    api.setup()
    rf = api.rf
    d = _inputs(api)
    counts = rf.scatter_count(indices=d["idx"], indices_dim=d["t"])
    got = counts.copy_transpose([api.batch_dim, d["f"]]).raw_tensor
    for b, n in enumerate(LENS):
        want = torch.bincount(d["idx"].raw_tensor[b, :n].long(), minlength=6)
        assert torch.equal(got[b].long(), want), (b, got[b], want)
    packed, pdim = rf.pack_padded(d["x"], dims=[api.batch_dim, d["t"]])
    assert packed.raw_tensor.shape[0] == sum(LENS)
    unpacked = rf.pad_packed(packed, in_dim=pdim, dims=[api.batch_dim, d["t"]])
    a = P.masked(P.to_numpy_bt(api, unpacked, [api.batch_dim, d["t"], d["f"]]), LENS)
    b = P.masked(d["x"].raw_tensor.numpy(), LENS)
    assert numpy.array_equal(a, b)


def test_complex_helpers():
    api = P.ours()
    api.setup()
    rf = api.rf
    pair = api.Dim(2, name="pair")
    f = api.Dim(5, name="f")
    x = api.tensor("x", [f, pair], numpy.arange(10, dtype="float32").reshape(5, 2))
    c = rf.real_as_complex(x, pair_dim=pair)
    assert c.dims == (f,) and c.raw_tensor.dtype == torch.complex64 and complex(c.raw_tensor[2]) == complex(4, 5)
    r, out_pair = rf.complex_as_real(c)
    assert out_pair.dimension == 2 and torch.equal(r.raw_tensor, x.raw_tensor)
    m = rf.make_complex(x.copy_with_raw(x.raw_tensor)[..., None] if False else api.tensor("re", [f], numpy.ones(5, "float32")),
                        api.tensor("im", [f], numpy.full(5, 2.0, "float32")))
    assert complex(m.raw_tensor[0]) == complex(1, 2)


def test_expand_make_non_empty():
    api = P.ours()
    api.setup()
    rf = api.rf
    t0 = api.time_dim([0, 0], name="empty")
    f = api.Dim(3, name="f")
    x = api.tensor("x", [api.batch_dim, t0, f], numpy.zeros((2, 0, 3), "float32"))
    y, t1 = rf.expand_make_non_empty(x, axis=t0)
    assert y.raw_tensor.shape == (2, 1, 3) and float(y.raw_tensor.abs().sum()) == 0.0
    d = _inputs(api)
    same, ax = rf.expand_make_non_empty(d["x"], axis=d["t"])
    assert same is d["x"] and ax is d["t"]


def test_amp_policy_casts():
    api = P.ours()
    api.setup()
    rf = api.rf
    d = _inputs(api)
    assert rf.get_amp_policy() is None and rf.amp_cast_compute(d["x"]) is d["x"]
    with rf.set_amp_policy_ctx("bfloat16"):
        assert rf.get_amp_policy() == rf.AmpPolicy(compute_dtype="bfloat16")
        a, i, n = rf.amp_cast_compute(d["x"], d["idx"], None)
        assert a.dtype == "bfloat16" and i is d["idx"] and n is None
        assert rf.amp_cast_float32(a).dtype == "float32"
    assert rf.get_amp_policy() is None
    with pytest.raises(ValueError):
        rf.AmpPolicy(compute_dtype="int32")


def test_static_traceable_flag_and_generation():
    rf = P.ours().rf
    g0 = rf.static_traceable_generation()
    assert not rf.is_static_traceable()
    with rf.set_static_traceable_ctx():
        assert rf.is_static_traceable() and rf.static_traceable_generation() == g0 + 1
        with rf.set_static_traceable_ctx(True):
            assert rf.static_traceable_generation() == g0 + 1  # no off -> on transition
    assert not rf.is_static_traceable()
    with rf.set_static_traceable_ctx():
        assert rf.static_traceable_generation() == g0 + 2


def test_parameter_copy_behaviour_and_default_dtype_ctx():
    import copy

    api = P.ours()
    rf = api.rf
    lin = rf.Linear(api.Dim(3, name="i"), api.Dim(2, name="o"))
    c1 = copy.deepcopy(lin)
    assert c1.weight is not lin.weight
    with rf.set_parameter_copy_behavior_ctx("share"):
        c2 = copy.deepcopy(lin)
    assert c2.weight is lin.weight
    with rf.set_default_float_dtype_ctx("float64"):
        assert rf.get_default_float_dtype() == "float64"
        assert rf.Parameter([api.Dim(2, name="p")]).dtype == "float64"
    assert rf.get_default_float_dtype() == "float32"


def test_step_based_seeds_repeat_after_reset():
    rf = P.ours().rf
    rf.reset_step_random_state()
    a = [int(rf.get_static_step_based_seed()) for _ in range(3)]
    rf.reset_step_random_state()
    b = [int(rf.get_static_step_based_seed()) for _ in range(3)]
    assert a == b and len(set(a)) == 3
    assert rf.get_static_step_based_seed(size=4).shape == (4,)


def test_conv_out_length_helpers():
    api = P.ours()
    api.setup()
    rf = api.rf
    assert rf.calc_conv_out_length(10, filter_size=3, stride=2, padding="same") == 5
    assert rf.calc_conv_out_length(10, filter_size=3, stride=2, padding="valid") == 4
    assert rf.calc_conv_out_length(10, filter_size=3, stride=1, padding=1) == 10
    assert rf.calc_conv_out_length(2, filter_size=5, stride=1, padding="valid") == 0
    t = api.time_dim(LENS)
    out = rf.calc_conv_out_length(t, filter_size=3, stride=2, padding="valid")
    assert out.dyn_size_ext.raw_tensor.tolist() == [4, 2, 1]
    assert rf.calc_transposed_conv_out_length(5, filter_size=3, padding="valid", stride=2) == 11
    assert rf.calc_transposed_conv_out_length(5, filter_size=2, padding="valid", stride=2) == 10
    assert rf.calc_transposed_conv_out_length(5, filter_size=3, padding="same", stride=2) == 10
    dims = rf.make_transposed_conv_out_spatial_dims([t], filter_size=3, padding="valid", strides=2)
    assert dims[0].dyn_size_ext.raw_tensor.tolist() == [19, 13, 7]


def test_run_ctx_step_tensor_and_misc_api():
    api = P.ours()
    rf = api.rf
    rf.init_train_step_run_ctx(train_flag=False, step=17, epoch=3)
    assert int(rf.get_run_ctx_step().raw_tensor) == 17
    assert rf.get_default_dim_size_device() == "cpu"
    assert rf.get_selected_backend() == "torch" and rf.is_backend_raw_tensor_dim_tag_independent()
    assert rf.get_raw_tensor_type() is torch.Tensor
    with pytest.raises(NotImplementedError):
        rf.select_backend("tensorflow")
    x = api.tensor("x", [api.Dim(2, name="d")], numpy.ones(2, "float32"))
    assert rf.get_tensor_dependencies(x) == [] and rf.walk_tensor_consumers(x) == [x]
    rf.assert_(True, "fine")
    with pytest.raises(AssertionError):
        rf.assert_(False, "boom")
    rf.assert_(x > 0, "all positive")
    assert rf.batch_norm_distributed_default() is False
