"""Dataset API, sequence orderings, partition epochs, batching pipeline (reference: returnn/datasets/basic.py, torch/data/pipeline.py)"""

import numpy
import pytest
from returnn_b200.datasets.basic import init_dataset, Dataset
from returnn_b200.datasets.generating import Task12AXDataset, StaticDataset, DummyGenericDataset


def _all_seqs(ds, epoch=1):
    ds.init_seq_order(epoch=epoch)
    seq, out = 0, []
    while ds.is_less_than_num_seqs(seq):
        ds.load_seqs(seq, seq + 1)
        out.append((ds.get_tag(seq), ds.get_data(seq, "data"), ds.get_data(seq, "classes")))
        seq += 1
    return out


def test_task12ax_deterministic_and_shapes():
    ds = init_dataset({"class": "Task12AXDataset", "num_seqs": 20, "fixed_random_seed": 3})
    a = _all_seqs(ds, 1)
    b = _all_seqs(ds, 1)
    assert len(a) == 20
    for (ta, xa, ya), (tb, xb, yb) in zip(a, b):
        assert ta == tb and numpy.array_equal(xa, xb) and numpy.array_equal(ya, yb)
        assert xa.shape[1] == 9 and xa.shape[0] == ya.shape[0] and ya.dtype == numpy.int32
    assert ds.get_data_dim("data") == 9 and ds.get_data_dim("classes") == 2


def _static(n=12, seq_ordering="default", **kw):
    rng = numpy.random.RandomState(0)
    data = [{"data": rng.randn(int(l), 3).astype("float32"), "classes": rng.randint(0, 5, (int(l),)).astype("int32")}
            for l in rng.randint(2, 30, n)]
    ds = StaticDataset(data=data, output_dim={"data": (3, 2), "classes": (5, 1)}, seq_ordering=seq_ordering, **kw)
    ds.initialize()
    return ds, data


@pytest.mark.parametrize("ordering", ["default", "reverse", "sorted", "sorted_reverse", "random", "laplace:3", "sort_bin_shuffle:.3"])
def test_seq_orderings_are_permutations(ordering):
    ds, data = _static(seq_ordering=ordering)
    seqs = _all_seqs(ds, 1)
    lens = [x.shape[0] for _, x, _ in seqs]
    assert sorted(lens) == sorted(d["data"].shape[0] for d in data)
    if ordering == "sorted":
        assert lens == sorted(lens)
    if ordering == "sorted_reverse":
        assert lens == sorted(lens, reverse=True)
    if ordering == "random":
        lens2 = [x.shape[0] for _, x, _ in _all_seqs(ds, 2)]
        assert sorted(lens2) == sorted(lens)  # another epoch, another order of the same data


def test_partition_epoch_covers_everything_once():
    ds, data = _static(n=10, partition_epoch=3)
    tags = []
    for ep in (1, 2, 3):
        tags += [t for t, _, _ in _all_seqs(ds, ep)]
    assert sorted(tags) == sorted("seq-%i" % i for i in range(10))
    assert [t for t, _, _ in _all_seqs(ds, 4)] == [t for t, _, _ in _all_seqs(ds, 1)]


def test_dummy_generic_dataset_from_extern_data():
    from returnn_b200.tensor import Dim, batch_dim

    t = Dim(None, name="time")
    ds = DummyGenericDataset({"data": {"dims": (batch_dim, t, Dim(7, name="f")), "dtype": "float32"},
                              "classes": {"dims": (batch_dim, t), "sparse_dim": Dim(4, name="c"), "dtype": "int32"}}, num_seqs=5, seq_lens=11)
    ds.initialize()
    seqs = _all_seqs(ds, 1)
    assert len(seqs) == 5 and seqs[0][1].shape == (11, 7) and seqs[0][2].max() < 4


def test_batching_pipeline_respects_frame_budget():
    from returnn_b200.torch.data import pipeline, returnn_dataset_wrapper

    ds, data = _static(n=40)
    wrapped = returnn_dataset_wrapper.ReturnnDatasetIterDataPipe(ds, reset_callback=lambda: ds.init_seq_order(epoch=1))
    batches = pipeline.BatchingIterDataPipe(wrapped, batch_size=60, max_seqs=8)
    n_seqs = 0
    for batch in batches:
        assert len(batch) <= 8
        max_len = max(b["data"].shape[0] for b in batch)
        assert max_len * len(batch) <= 60 or len(batch) == 1
        n_seqs += len(batch)
        coll = pipeline.collate_batch(batch)
        assert coll["data"].shape[0] == len(batch) and coll["data"].shape[1] == max_len
        assert coll["data:seq_len"].tolist() == [b["data"].shape[0] for b in batch]
    assert n_seqs == 40


def test_vocabulary_roundtrip(tmp_path):
    from returnn_b200.datasets.util.vocabulary import Vocabulary

    fn = tmp_path / "vocab.txt"
    fn.write_text("{'<s>': 0, '</s>': 1, 'a': 2, 'b': 3, '<unk>': 4}")
    v = Vocabulary(str(fn), unknown_label="<unk>")
    assert v.num_labels == 5
    ids = v.get_seq("a b c")
    assert ids == [2, 3, 4]
    assert v.get_seq_labels(ids) == "a b <unk>"
