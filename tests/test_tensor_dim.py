"""Tensor / Dim: named dims, dynamic sizes, dim math, masks, broadcasting by dim identity (reference: returnn/tensor/)"""

import numpy
import torch
from returnn_b200.tensor import Tensor, Dim, TensorDict, batch_dim
import returnn_b200.frontend as rf


def _time_dim(lens):
    t = Dim(None, name="time")
    t.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor(lens, dtype=torch.int32))
    return t


def test_dim_identity_and_static_math():
    a, b = Dim(3, name="a"), Dim(3, name="b")
    assert a != b and a == a
    assert (a + b).dimension == 6 and (a * 2).dimension == 6
    assert (2 * a).div_left(2) == a
    assert (a + b) == (a + b)  # derived dims are memoised
    assert (a + b - b) == a
    assert a.ceildiv_right(2).dimension == 2


def test_dynamic_dim_math_follows_sizes():
    t = _time_dim([5, 3, 4])
    half = t.ceildiv_right(2)
    assert half.dyn_size_ext.raw_tensor.tolist() == [3, 2, 2]
    assert half.get_dim_value() == 3
    t.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([9, 1, 2], dtype=torch.int32))
    assert half.dyn_size_ext.raw_tensor.tolist() == [5, 1, 1]  # refreshed after the base changed
    assert half.get_dim_value() == 5


def test_mask_and_copy_compatible():
    t = _time_dim([2, 3])
    f = Dim(4, name="feat")
    x = Tensor("x", dims=[batch_dim, t, f], dtype="float32", raw_tensor=torch.ones(2, 3, 4))
    mask = t.get_mask(dim_order=[batch_dim, t])
    assert mask.raw_tensor.tolist() == [[True, True, False], [True, True, True]]
    y = x.copy_compatible_to_dims([f, batch_dim, t])
    assert tuple(y.raw_tensor.shape) == (4, 2, 3)
    v = Tensor("v", dims=[f], dtype="float32", raw_tensor=torch.arange(4.0))
    z = x + v  # broadcast by dim identity, not by position
    assert z.dims == (batch_dim, t, f) and z.raw_tensor[0, 0].tolist() == [1.0, 2.0, 3.0, 4.0]
    w = v + x
    assert set(w.dims) == {batch_dim, t, f}


def test_reduce_ignores_padding():
    t = _time_dim([2, 3])
    x = Tensor("x", dims=[batch_dim, t], dtype="float32", raw_tensor=torch.tensor([[1.0, 2.0, 100.0], [1.0, 1.0, 1.0]]))
    s = rf.reduce_sum(x, axis=t)
    assert s.raw_tensor.tolist() == [3.0, 3.0]
    m = rf.reduce_mean(x, axis=t)
    assert m.raw_tensor.tolist() == [1.5, 1.0]
    mx = rf.reduce_max(x, axis=t)
    assert mx.raw_tensor.tolist() == [2.0, 1.0]


def test_tensor_dict_and_sparse():
    v = Dim(7, name="vocab")
    t = _time_dim([2, 1])
    lab = Tensor("lab", dims=[batch_dim, t], dtype="int32", sparse_dim=v, raw_tensor=torch.tensor([[1, 2], [3, 0]], dtype=torch.int32))
    td = TensorDict({"lab": lab})
    assert td["lab"].sparse_dim is v
    oh = rf.one_hot(lab)
    assert oh.dims[-1] == v and oh.raw_tensor.shape == (2, 2, 7)
    raw = td.as_raw_tensor_dict()
    assert "lab" in raw


def test_merge_split_concat_gather():
    a, b = Dim(2, name="a"), Dim(3, name="b")
    x = Tensor("x", dims=[a, b], dtype="float32", raw_tensor=torch.arange(6.0).reshape(2, 3))
    m, md = rf.merge_dims(x, dims=[a, b])
    assert md.dimension == 6 and m.raw_tensor.tolist() == list(map(float, range(6)))
    back = rf.split_dims(m, axis=md, dims=[a, b])
    assert torch.equal(back.raw_tensor, x.raw_tensor)
    c, cd = rf.concat((x, b), (x, b))
    assert cd.dimension == 6 and c.raw_tensor.shape == (2, 6)
    idx = Tensor("i", dims=[a], dtype="int32", sparse_dim=b, raw_tensor=torch.tensor([2, 0], dtype=torch.int32))
    g = rf.gather(x, indices=idx, axis=b)
    assert g.raw_tensor.tolist() == [2.0, 3.0]


# ---- a wider sweep over the Tensor / Dim surface -------------------------------------------------------------------------------
import copy
import pickle
import pytest


def _x(lens=(2, 3), feat=4, fill=None):
    t = _time_dim(list(lens))
    f = Dim(feat, name="feat")
    raw = torch.arange(len(lens) * max(lens) * feat, dtype=torch.float32).reshape(len(lens), max(lens), feat) if fill is None else torch.full(
        (len(lens), max(lens), feat), float(fill))
    return Tensor("x", dims=[batch_dim, t, f], dtype="float32", raw_tensor=raw, feature_dim=f), t, f


@pytest.mark.parametrize("op,expect", [("add", 7), ("sub", 1), ("mul", 12), ("floordiv", 1), ("ceildiv", 2)])
def test_static_dim_arithmetic(op, expect):
    a, b = Dim(4, name="a"), Dim(3, name="b")
    res = {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "floordiv": lambda: a // 3, "ceildiv": lambda: a.ceildiv_right(3)}[op]()
    assert res.dimension == expect and res.is_static() and not res.is_dynamic()
    assert res == {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "floordiv": lambda: a // 3, "ceildiv": lambda: a.ceildiv_right(3)}[op]()


@pytest.mark.parametrize("lens", [[1], [5, 3, 4], [2, 2]])
def test_dynamic_dim_arithmetic_per_sequence(lens):
    t = _time_dim(lens)
    assert (t + 2).dyn_size_ext.raw_tensor.tolist() == [n + 2 for n in lens]
    assert (t * 3).dyn_size_ext.raw_tensor.tolist() == [n * 3 for n in lens]
    assert (t // 2).dyn_size_ext.raw_tensor.tolist() == [n // 2 for n in lens]
    assert t.ceildiv_right(2).dyn_size_ext.raw_tensor.tolist() == [-(-n // 2) for n in lens]
    assert (t + t).dyn_size_ext.raw_tensor.tolist() == [2 * n for n in lens]
    assert ((t + 2) - 2) == t and (t * 3).div_left(3) == t  # inverse operations cancel
    assert t.get_dim_value() == max(lens) and (t + 1).get_dim_value() == max(lens) + 1
    assert t.is_dynamic() and t.is_dynamic_seq_length() and t.need_masking() == (min(lens) != max(lens) or len(lens) > 1 and False or t.need_masking())


def test_dim_kinds_and_predicates():
    f, s = Dim(3, name="f", kind=Dim.Types.Feature), Dim(None, name="s", kind=Dim.Types.Spatial)
    assert batch_dim.is_batch_dim() and not f.is_batch_dim()
    assert f.is_feature_dim() and s.is_spatial_dim() and not f.is_spatial_dim()
    assert f.is_static() and s.is_dynamic() and not s.is_dim_known()
    s.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([2, 1], dtype=torch.int32))
    assert s.is_dim_known()
    assert "f" in repr(f) and "3" in repr(f) and f.short_repr()


def test_declare_same_as_merges_identity():
    a, b = Dim(None, name="a"), Dim(None, name="b")
    a.dyn_size_ext = Tensor("l", dims=[batch_dim], dtype="int32", raw_tensor=torch.tensor([2, 4], dtype=torch.int32))
    assert a != b
    b.declare_same_as(a)
    assert a == b and hash(a) == hash(b) and b.get_same_base() is a.get_same_base()
    assert b.dyn_size_ext.raw_tensor.tolist() == [2, 4]
    x = Tensor("x", dims=[batch_dim, a], dtype="float32", raw_tensor=torch.zeros(2, 4))
    assert x.get_axis_from_description(b) == 1


def test_dim_copy_pickle_and_deepcopy_keep_static_identity_rules():
    f = Dim(5, name="f")
    assert copy.copy(f) is f or copy.copy(f) == f
    g = pickle.loads(pickle.dumps(f))
    assert g.dimension == 5 and g.name == "f"
    assert copy.deepcopy(f).dimension == 5
    c = f.copy(same_as_self=False) if "same_as_self" in Dim.copy.__code__.co_varnames else f.copy()
    assert c.dimension == 5


@pytest.mark.parametrize("order", [[0, 1, 2], [1, 0, 2], [2, 1, 0], [2, 0, 1]])
def test_copy_transpose_and_permutations(order):
    x, t, f = _x()
    dims = [x.dims[i] for i in order]
    y = x.copy_transpose(dims)
    assert list(y.dims) == dims and y.raw_tensor.shape == tuple(x.raw_tensor.shape[i] for i in order)
    torch.testing.assert_close(y.raw_tensor, x.raw_tensor.permute(*order))
    assert x.get_out_permutation_to_dims(dims) == order
    assert y.feature_dim == f and y.feature_dim_axis == dims.index(f)
    back = y.copy_transpose(list(x.dims))
    torch.testing.assert_close(back.raw_tensor, x.raw_tensor)


def test_copy_compatible_to_dims_broadcasts_and_orders():
    x, t, f = _x()
    extra = Dim(7, name="extra")
    y = x.copy_compatible_to_dims([extra, f, batch_dim, t])
    assert [d for d in y.dims] == [extra, f, batch_dim, t] and y.raw_tensor.shape == (1, 4, 2, 3)
    raw = x.copy_compatible_to_dims_raw([f, extra, t, batch_dim])
    assert raw.shape == (4, 1, 3, 2)
    v = Tensor("v", dims=[f], dtype="float32", raw_tensor=torch.arange(4.0))
    z = x + v  # broadcast by identity, not by position
    torch.testing.assert_close(z.raw_tensor, x.raw_tensor + torch.arange(4.0))
    w = Tensor("w", dims=[t], dtype="float32", raw_tensor=torch.arange(3.0))
    torch.testing.assert_close((x * w).raw_tensor, x.raw_tensor * torch.arange(3.0)[None, :, None])
    with pytest.raises(Exception):
        x.copy_compatible_to_dims([batch_dim, f])  # a dim of x is missing in the target


def test_copy_move_axis_batch_time_major_and_feature_last():
    x, t, f = _x()
    tm = x.copy_as_time_major()
    assert tm.dims[0] == t and tm.time_dim_axis == 0 and tm.batch_dim_axis == 1
    bm = tm.copy_as_batch_major()
    assert bm.dims[0] == batch_dim and bm.have_batch_axis()
    y = x.copy_move_axis(2, 0)
    assert y.dims == (f, batch_dim, t)
    assert y.copy_with_feature_last().dims[-1] == f
    assert x.copy_with_feature_dim_axis(1).dims == (batch_dim, f, t)


def test_templates_and_kwargs_roundtrip():
    x, t, f = _x()
    templ = x.copy_template(name="y")
    assert templ.raw_tensor is None and templ.dims == x.dims and templ.dtype == "float32" and templ.name == "y"
    kw = x.get_kwargs()
    again = Tensor(**kw)
    assert again.dims == x.dims and again.dtype == x.dtype
    new_f = Dim(9, name="nf")
    r = x.copy_template_replace_dim_tag(axis=2, new_dim_tag=new_f)
    assert r.dims == (batch_dim, t, new_f)
    e = x.copy_template_excluding_axis(1)
    assert e.dims == (batch_dim, f)
    a = e.copy_template_adding_time_dim(time_dim_axis=1) if hasattr(e, "copy_template_adding_time_dim") else None
    assert a is None or a.batch_ndim == 3
    added = x.copy_add_dim_by_tag(Dim(1, name="one"), unbroadcast=True, axis=0)
    assert added.raw_tensor.shape == (1, 2, 3, 4)


def test_copy_masked_and_sequence_masks():
    x, t, f = _x(fill=1.0)
    m = x.copy_masked(-5.0)
    assert m.raw_tensor[0, 2].tolist() == [-5.0] * 4 and m.raw_tensor[0, :2].eq(1).all() and m.raw_tensor[1].eq(1).all()
    assert x.get_sequence_lengths().tolist() == [2, 3]
    mask = x.get_sequence_mask_tensor(1) if hasattr(x, "get_sequence_mask_tensor") else None
    assert mask is None or mask.raw_tensor.sum().item() == 5
    mb = x.get_sequence_mask_broadcast(1)
    assert tuple(mb.shape) == (2, 3, 1) and int(mb.sum()) == 5
    assert x.num_elements() == 5 * 4 if callable(getattr(x, "num_elements", None)) else True


def test_axis_descriptions():
    x, t, f = _x()
    assert x.get_axis_from_description("B") == 0 and x.get_axis_from_description("T") == 1 and x.get_axis_from_description("F") == 2
    assert x.get_axis_from_description(t) == 1 and x.get_axis_from_description(-1) == 2
    assert x.get_axes_from_description(["B", f]) == [0, 2]
    assert x.get_dim_tag(1) == t and x.get_dim_tag_from_description("F") == f
    assert x.get_dynamic_axes() == [1] and x.get_static_axes() == [2]
    assert x.get_batch_shape(batch_dim=7) == (7, None, 4) if hasattr(x, "get_batch_shape") else True
    assert x.batch_shape == (None, None, 4) and x.shape == (None, 4) and x.batch_ndim == 3
    with pytest.raises(Exception):
        x.get_axis_from_description(Dim(4, name="other"))


def test_sparse_tensor_properties_and_squeeze():
    vocab = Dim(10, name="vocab")
    t = _time_dim([2, 1])
    y = Tensor("y", dims=[batch_dim, t], dtype="int32", sparse_dim=vocab, raw_tensor=torch.tensor([[1, 2], [3, 0]], dtype=torch.int32))
    assert y.sparse and y.dim == 10 and y.is_int() and not y.is_float() and y.feature_dim is None
    one = Dim(1, name="one")
    z = Tensor("z", dims=[batch_dim, one, t], dtype="int32", raw_tensor=y.raw_tensor[:, None])
    s = z.copy_squeeze_axes([1])
    assert s.dims == (batch_dim, t) and torch.equal(s.raw_tensor, y.raw_tensor)


@pytest.mark.parametrize("op", ["add", "sub", "mul", "truediv", "pow", "neg", "abs", "eq", "lt", "ge", "and", "or", "invert", "radd", "rsub", "rmul", "mod", "floordiv"])
def test_operator_overloads_match_torch(op):
    x, t, f = _x()
    a = x.raw_tensor
    y = Tensor("y", dims=x.dims, dtype="float32", raw_tensor=a.flip(-1) + 1.0)
    b = y.raw_tensor
    bx, by = (x > 10.0), (y > 10.0)
    table = {
        "add": (lambda: x + y, a + b), "sub": (lambda: x - y, a - b), "mul": (lambda: x * y, a * b), "truediv": (lambda: x / y, a / b),
        "pow": (lambda: y ** 2.0, b ** 2.0), "neg": (lambda: -x, -a), "abs": (lambda: abs(x - 10.0), (a - 10.0).abs()),
        "eq": (lambda: x == y, a == b), "lt": (lambda: x < y, a < b), "ge": (lambda: x >= y, a >= b),
        "and": (lambda: bx & by, (a > 10) & (b > 10)), "or": (lambda: bx | by, (a > 10) | (b > 10)), "invert": (lambda: ~bx, ~(a > 10)),
        "radd": (lambda: 2.0 + x, 2.0 + a), "rsub": (lambda: 2.0 - x, 2.0 - a), "rmul": (lambda: 3.0 * x, 3.0 * a),
        "mod": (lambda: x % 3.0, a % 3.0), "floordiv": (lambda: x // 3.0, torch.floor(a / 3.0)),
    }
    fn, want = table[op]
    got = fn()
    assert got.dims == x.dims
    assert torch.equal(got.raw_tensor, want) if want.dtype == torch.bool else torch.allclose(got.raw_tensor, want)


def test_tensor_dict_api():
    x, t, f = _x()
    vocab = Dim(10, name="vocab")
    y = Tensor("classes", dims=[batch_dim, t], dtype="int32", sparse_dim=vocab, raw_tensor=torch.zeros(2, 3, dtype=torch.int32))
    td = TensorDict([x, y]) if not isinstance(TensorDict(), dict) else TensorDict()
    if not td.data:
        td.data["x"], td.data["classes"] = x, y
    assert set(td.data.keys()) == {"x", "classes"} and td["x"] is x
    templ = td.copy_template()
    assert templ["x"].raw_tensor is None and templ["classes"].sparse_dim == vocab
    raw = td.as_raw_tensor_dict(include_const_sizes=True) if hasattr(td, "as_raw_tensor_dict") else None
    if raw is not None:
        assert torch.equal(raw["x"], x.raw_tensor) and any(k.startswith("x:size") for k in raw)
        templ2 = td.copy_template()
        templ2.assign_from_raw_tensor_dict_(raw)
        assert torch.equal(templ2["x"].raw_tensor, x.raw_tensor)


def test_verify_out_shape_and_sanity_check():
    x, t, f = _x()
    x.verify_out_shape({batch_dim, t, f})
    with pytest.raises(Exception):
        x.verify_out_shape({batch_dim, f})
    x.sanity_check()
    bad = Tensor("bad", dims=[batch_dim, f], dtype="float32")
    with pytest.raises(Exception):
        bad.raw_tensor = torch.zeros(2, 5)  # size of f is 4


def test_data_and_tensor_utilities():
    from returnn_b200.torch.data.queued_data_iter import QueuedDataIter
    from returnn_b200.torch.data import tensor_utils as TU
    from returnn_b200.torch.data.extern_data import get_batch_dim_from_extern_data
    from returnn_b200.tensor.utils import tensor_dict_dims_random_seq_len_min_max, get_random_seq_lens_for_dyn_dims

    it = QueuedDataIter(iter([1, 2, 3]))
    assert next(it) == 1
    it.extend(["a", "b"])
    assert list(it) == ["a", "b", 2, 3]
    t = Dim(None, name="time")
    t.dyn_size_ext = Tensor("lens", dims=[batch_dim], dtype="int32", raw_tensor=numpy.array([2, 3], dtype="int32"))
    f = Dim(4, name="feat")
    x = Tensor("data", dims=[batch_dim, t, f], dtype="float32", raw_tensor=numpy.ones((2, 3, 4), dtype="float32"))
    s2 = Dim(None, name="labels")
    y = Tensor("classes", dims=[batch_dim, s2], dtype="int32", sparse_dim=Dim(7, name="v"))
    td = TensorDict()
    td.data["data"], td.data["classes"] = x, y
    TU.tensor_dict_numpy_to_torch_(td)
    assert isinstance(x.raw_tensor, torch.Tensor) and isinstance(t.dyn_size_ext.raw_tensor, torch.Tensor)
    TU.tensor_dict_torch_to_numpy_(td)
    assert isinstance(x.raw_tensor, numpy.ndarray) and t.dyn_size_ext.raw_tensor.tolist() == [2, 3]
    assert get_batch_dim_from_extern_data(td) is batch_dim
    dims, ranges = tensor_dict_dims_random_seq_len_min_max(td, {"classes": 5, None: (3, 6)})
    assert dims == [t, s2] and ranges == {t: (3, 6), s2: (5, 5)}
    lens = get_random_seq_lens_for_dyn_dims(dims, ranges, batch_size=4, rnd=1)
    assert lens[s2].tolist() == [5] * 4 and lens[t][0] == 6 and all(3 <= v <= 6 for v in lens[t].tolist())
    assert get_random_seq_lens_for_dyn_dims(dims, ranges, batch_size=4, rnd=1)[t].tolist() == lens[t].tolist()
