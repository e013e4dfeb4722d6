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


def _read_all(ds, epoch=1, keys=("data",)):
    ds.init_seq_order(epoch=epoch)
    i, out = 0, []
    while ds.is_less_than_num_seqs(i):
        ds.load_seqs(i, i + 1)
        out.append((ds.get_tag(i),) + tuple(ds.get_data(i, k) for k in keys))
        i += 1
    return out


def test_meta_and_concat_datasets(tmp_path):
    rng = numpy.random.RandomState(0)
    mk = lambda n: [{"data": rng.randn(int(l), 3).astype("float32"), "classes": rng.randint(0, 5, (int(l),)).astype("int32")} for l in rng.randint(2, 9, n)]
    a = {"class": "StaticDataset", "data": mk(6), "output_dim": {"data": (3, 2), "classes": (5, 1)}}
    b = {"class": "StaticDataset", "data": mk(6), "output_dim": {"data": (3, 2), "classes": (5, 1)}}
    meta = init_dataset({"class": "MetaDataset", "datasets": {"x": a, "y": b}, "data_map": {"data": ("x", "data"), "classes": ("y", "classes")},
                         "seq_order_control_dataset": "x"})
    seqs = _read_all(meta, keys=("data", "classes"))
    assert len(seqs) == 6 and seqs[0][1].shape == a["data"][0]["data"].shape and numpy.array_equal(seqs[0][2], b["data"][0]["classes"])
    assert len(_read_all(init_dataset({"class": "ConcatDataset", "datasets": [a, b]}))) == 12
    comb = init_dataset({"class": "CombinedDataset", "datasets": {"x": a, "y": b},
                         "data_map": {("x", "data"): "data", ("y", "data"): "data", ("x", "classes"): "classes"}, "seq_ordering": "random"})
    got = _read_all(comb, keys=("data", "classes"))
    assert len(got) == 12 and sum(1 for g in got if g[2].shape[0] == 0) == 6  # dataset y has no "classes": empty arrays
    lst = tmp_path / "seqs.txt"
    lst.write_text("seq-0;seq-1\nseq-2;seq-3;seq-4\n")
    cs = _read_all(init_dataset({"class": "ConcatSeqsDataset", "dataset": a, "seq_list_file": str(lst)}))
    assert [t for t, _ in cs] == ["seq-0;seq-1", "seq-2;seq-3;seq-4"]
    assert cs[0][1].shape[0] == a["data"][0]["data"].shape[0] + a["data"][1]["data"].shape[0]


def test_npz_writer_dataset_and_distribute_files(tmp_path):
    from returnn_b200.datasets.hdf import SimpleHDFWriter

    rng = numpy.random.RandomState(0)
    files = []
    for f in range(6):
        fn = str(tmp_path / ("part%i.npz" % f))
        files.append(fn)
        with SimpleHDFWriter(fn, dim=2, extra_type={"classes": (5, 1, "int32")}) as w:
            for i in range(3):
                n = 2 + f
                w.insert_seq(rng.randn(n, 2).astype("float32"), "f%i-s%i" % (f, i), extra={"classes": rng.randint(0, 5, (n,)).astype("int32")})
    one = _read_all(init_dataset({"class": "NpzDataset", "files": files[:2], "seq_ordering": "sorted_reverse"}), keys=("data", "classes"))
    assert len(one) == 6 and one[0][1].shape == (3, 2) and one[0][2].shape == (3,)
    seen = {}
    for rank in (0, 1):
        ds = init_dataset({"class": "DistributeFilesDataset", "files": files, "get_sub_epoch_dataset": lambda fs: {"class": "NpzDataset", "files": fs},
                           "partition_epoch": 3, "_distrib_info": {"rank": rank, "size": 2}})
        for ep in (1, 2, 3):
            for tag, _ in _read_all(ds, epoch=ep):
                seen.setdefault(tag, []).append((rank, ep))
    assert len(seen) == 18 and all(len(v) == 1 for v in seen.values())  # every sequence exactly once over ranks and sub-epochs


def test_postprocessing_lm_and_text(tmp_path):
    from returnn_b200.datasets.postprocessing import LaplaceOrdering

    def double(td, **_kw):
        td.data["data"].raw_tensor = td.data["data"].raw_tensor * 2
        return td

    ds = init_dataset({"class": "PostprocessingDataset", "dataset": {"class": "Task12AXDataset", "num_seqs": 10, "fixed_random_seed": 2},
                       "map_seq": double, "map_seq_stream": LaplaceOrdering(4)})
    seqs = _read_all(ds)
    lens = [x.shape[0] for _, x in seqs]
    assert len(lens) == 10 and lens[:4] == sorted(lens[:4]) and lens[4:8] == sorted(lens[4:8], reverse=True)
    assert max(x.max() for _, x in seqs) == 2.0
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("b a\nab\n\na b a b\n")
    syms = tmp_path / "syms.txt"
    syms.write_text("a\nb\n_\n[END]\n")
    lm = init_dataset({"class": "LmDataset", "corpus_file": str(corpus), "orth_symbols_file": str(syms), "word_end_symbol": "_", "seq_ordering": "sorted"})
    got = _read_all(lm)
    assert [x.tolist() for _, x in got] == [[0, 1, 3], [1, 2, 0, 3], [0, 2, 1, 2, 0, 2, 1, 3]]


def test_literal_parser_matches_ast():
    import ast
    from returnn_b200.utils.literal_py_to_pickle import literal_eval

    txt = "{'a': [1, 2.5, -3, 12345678901234567890, True, None], \"b\\n\": ('x', 'y',), 'c': {'d': 'caf\\u00e9'}, # comment\n 'e': [],}"
    assert literal_eval(txt) == ast.literal_eval(txt)


def test_rank_balanced_batching_equalises_real_frames():
    """the ranks of a step get disjoint batches with near-equal sums of sequence lengths"""
    import numpy
    from returnn_b200.torch.data.pipeline import balance_batches, BatchingIterDataPipe, RankBalancedBatchingIterDataPipe

    rng = numpy.random.RandomState(7)
    seqs = [{"data": numpy.zeros((int(rng.randint(300, 2001)), 2), dtype="float32"), "seq_idx": numpy.array(i)} for i in range(400)]
    budget, world = 40000, 4
    plain = list(BatchingIterDataPipe(seqs, batch_size=budget, max_seqs=200))
    groups = [plain[i: i + world] for i in range(0, len(plain) - world + 1, world)]
    spread_before, spread_after = [], []
    for g in groups:
        bal = balance_batches(g, length_key="data", max_seqs=200)
        assert sorted(int(s["seq_idx"]) for b in g for s in b) == sorted(int(s["seq_idx"]) for b in bal for s in b)
        for b in bal:
            assert b and len(b) <= 200
        real_before = [sum(s["data"].shape[0] for s in b) for b in g]
        real_after = [sum(s["data"].shape[0] for s in b) for b in bal]
        spread_before.append(max(real_before) / (sum(real_before) / world))
        spread_after.append(max(real_after) / (sum(real_after) / world))
    assert numpy.mean(spread_after) < 1.03 < numpy.mean(spread_before), (numpy.mean(spread_before), numpy.mean(spread_after))
    # the data pipe: every rank computes the same partition and keeps its own part
    per_rank = [list(RankBalancedBatchingIterDataPipe(seqs, batch_size=budget, max_seqs=200, length_key="data", rank=r, world=world)) for r in range(world)]
    assert len({len(x) for x in per_rank}) == 1 and len(per_rank[0]) == len(groups)
    for step in range(len(groups)):
        ids = [int(s["seq_idx"]) for r in range(world) for s in per_rank[r][step]]
        assert len(ids) == len(set(ids)) == sum(len(b) for b in groups[step])
