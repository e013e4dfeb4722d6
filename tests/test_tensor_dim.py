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
