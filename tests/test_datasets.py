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


def _write_stream_file(path, rng, n_seqs=7, n_classes=3, first=0):
    from returnn_b200.datasets.hdf import NextGenHDFWriter

    seqs = {}
    with NextGenHDFWriter(str(path)) as w:
        w.add_stream("features", "feature_sequence")
        w.add_stream("words", "sparse", feature_names=["w%i" % i for i in range(n_classes)])
        w.add_stream("align", "segment_alignment", feature_names=["a", "b", "c", "d"])
        for i in range(n_seqs):
            t = int(rng.randint(3, 9))
            feat = rng.standard_normal((t, 4)).astype("float32")
            word = numpy.array([(first + i) % n_classes], dtype="int32")
            segs = numpy.array([[1, 2], [3, t - 2]], dtype="int32")
            name = "corpus/rec%i/%i" % (first, i)
            w.add_seq(name, {"features": feat, "words": word, "align": segs})
            seqs[name] = (feat, word, segs)
    return seqs


def test_next_gen_hdf_dataset_streams(tmp_path):
    """stream-layout files: every stream is a data key, several files, sorted order, the segment alignment expanded per frame"""
    from returnn_b200.datasets.hdf import NextGenHDFDataset

    rng = numpy.random.RandomState(3)
    seqs = _write_stream_file(tmp_path / "a.hdf", rng)
    seqs.update(_write_stream_file(tmp_path / "b.hdf", rng, n_seqs=4, first=1))
    ds = NextGenHDFDataset("features", files=[str(tmp_path / "a.hdf"), str(tmp_path / "b.hdf")], seq_ordering="sorted")
    ds.initialize()
    assert ds.num_inputs == 4 and ds.num_outputs["words"] == [3, 1] and ds.num_outputs["align"] == [4, 1] and ds.get_data_dtype("data") == "float32"
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 11
    lens = []
    for i in range(ds.num_seqs):
        ds.load_seqs(i, i + 1)
        tag = ds.get_tag(i)
        feat, word, segs = seqs[tag]
        assert numpy.array_equal(ds.get_data(i, "data"), feat) and numpy.array_equal(ds.get_data(i, "features"), feat)
        assert numpy.array_equal(ds.get_data(i, "words"), word)
        al = ds.get_data(i, "align").reshape(-1, 2)
        t = feat.shape[0]
        assert al.shape[0] == t and al[:2, 0].tolist() == [1, 1] and set(al[2:, 0].tolist()) == {3}
        assert al[:, 1].tolist() == [0, 1] + [0] * (t - 3) + [1]
        lens.append(t)
    assert lens == sorted(lens)


def test_siamese_hdf_dataset_triplets(tmp_path):
    """anchor / same-label / other-label triplets, re-drawn per epoch"""
    from returnn_b200.datasets.hdf import SiameseHDFDataset

    rng = numpy.random.RandomState(4)
    _write_stream_file(tmp_path / "s.hdf", rng, n_seqs=12, n_classes=3)
    ds = SiameseHDFDataset("features", seq_label_stream="words", files=[str(tmp_path / "s.hdf")], fixed_random_seed=7)
    ds.initialize()
    picks = []
    for epoch in (1, 2):
        ds.init_seq_order(epoch=epoch)
        row = []
        for i in range(ds.num_seqs):
            ds.load_seqs(i, i + 1)
            w0, w1, w2 = (int(ds.get_data(i, "words_%i" % k)[0]) for k in range(3))
            assert w0 == w1 != w2
            assert ds.get_data(i, "words_all").tolist() == [w0, w1, w2]
            assert numpy.array_equal(ds.get_data(i, "data"), ds.get_data(i, "features_0"))
            assert not numpy.array_equal(ds.get_data(i, "features_0"), ds.get_data(i, "features_1"))  # 4 sequences per class: never itself
            row.append((ds.get_data(i, "features_1").tobytes(), ds.get_data(i, "features_2").tobytes()))
        picks.append(row)
    assert picks[0] != picks[1]
    assert ds.get_data_dim("features_2") == 4 and not ds.is_data_sparse("features_1") and ds.is_data_sparse("words_0")


def test_simple_hdf_writer_and_hdf_dataset_roundtrip(tmp_path):
    """SimpleHDFWriter -> HDFDataset through the HDF container (the stand-in where h5py is missing)"""
    from returnn_b200.datasets.hdf import SimpleHDFWriter, HDFDataset

    fn = str(tmp_path / "d.hdf")
    rng = numpy.random.RandomState(1)
    seqs = []
    with SimpleHDFWriter(fn, dim=3, ndim=2, extra_type={"classes": (5, 1, "int32")}) as w:
        for i in range(5):
            t = 2 + i
            x = rng.standard_normal((t, 3)).astype("float32")
            c = rng.randint(0, 5, size=(t,)).astype("int32")
            w.insert_seq(x, "seq-%i" % i, extra={"classes": c})
            seqs.append((x, c))
    ds = HDFDataset(files=[fn])
    ds.initialize()
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 5 and ds.get_data_dim("classes") == 5 and ds.is_data_sparse("classes")
    for i in range(5):
        ds.load_seqs(i, i + 1)
        assert ds.get_tag(i) == "seq-%i" % i
        assert numpy.array_equal(ds.get_data(i, "data"), seqs[i][0]) and numpy.array_equal(ds.get_data(i, "classes"), seqs[i][1])


def _write_wav(path, samples, rate=16000):
    import wave

    with wave.open(str(path), "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(rate)
        w.writeframes((numpy.clip(samples, -1, 1) * 32767).astype("<i2").tobytes())


def test_clustering_and_chunk_shuffle_datasets(tmp_path):
    from returnn_b200.datasets.basic import init_dataset

    cmap = tmp_path / "cluster.map"
    cmap.write_text('<?xml version="1.0"?>\n<coprus-key-map>\n' + "".join('<map-item key="seq-%i" value="%i"/>\n' % (i, i % 3) for i in range(12)) + "</coprus-key-map>\n")
    ds = init_dataset({"class": "ClusteringDataset", "dataset": {"class": "DummyDataset", "input_dim": 3, "output_dim": 4, "num_seqs": 12, "seq_len": 5},
                       "cluster_map_file": str(cmap), "n_clusters": 3})
    ds.init_seq_order(epoch=1)
    assert "cluster_idx" in ds.get_data_keys() and ds.get_data_dim("cluster_idx") == 3 and ds.is_data_sparse("cluster_idx")
    for i in range(12):
        ds.load_seqs(i, i + 1)
        assert ds.get_data(i, "cluster_idx").tolist() == [i % 3] and ds.get_data(i, "data").shape == (5, 3)
    sub = {"class": "DummyDataset", "input_dim": 2, "output_dim": 3, "num_seqs": 9, "seq_len": 20, "chunking": "6:6"}
    cs = init_dataset({"class": "ChunkShuffleDataset", "dataset": sub, "chunk_shuffle_cache": 8, "batch_gen_batch_size": 1000, "batch_gen_max_seqs": 1})
    orders = []
    for epoch in (1, 2):
        cs.init_seq_order(epoch=epoch)
        tags, frames, i = [], 0, 0
        while cs.is_less_than_num_seqs(i):
            cs.load_seqs(i, i + 1)
            tags.append(cs.get_tag(i))
            x = cs.get_data(i, "data")
            assert 0 < x.shape[0] <= 6 and cs.get_data(i, "classes").shape[0] == x.shape[0]
            frames += x.shape[0]
            i += 1
        assert frames == 9 * 20 and len(tags) == 9 * 4 and len(set(tags)) == len(tags)
        orders.append(tags)
    running = [int(t.rsplit(".", 1)[1]) for t in orders[0]]
    assert running != sorted(running) and sorted(running) == list(range(36))  # shuffled, every chunk exactly once
    assert orders[0] != orders[1]


def test_stereo_hdf_dataset_with_bundle_and_normalization(tmp_path):
    from returnn_b200.utils.h5_shim import get_h5py
    from returnn_b200.datasets.stereo import StereoHdfDataset, DatasetWithTimeContext
    from returnn_b200.datasets.normalization_data import NormalizationData
    from returnn_b200.datasets.bundle_file import BundleFile

    h5py = get_h5py()
    rng = numpy.random.RandomState(0)
    ref = {}
    files = []
    for fi in range(2):
        fn = tmp_path / ("part%i.hdf" % fi)
        with h5py.File(str(fn), "w") as f:
            gi, go = f.create_group("inputs"), f.create_group("outputs")
            for j in range(3):
                t = 4 + j
                x, y = rng.standard_normal((t, 3)) + 2.0, rng.standard_normal((t, 2)) - 1.0
                gi.create_dataset(str(j), data=x)
                go.create_dataset(str(j), data=y)
                ref[(fi, j)] = (x, y)
        files.append(str(fn))
    bundle = tmp_path / "all.bundle"
    bundle.write_text("\n".join(files) + "\n\n")
    assert BundleFile(str(bundle)).number_of_dataset_files == 2
    norm_fn = str(tmp_path / "norm.hdf")
    NormalizationData.create_normalization_file(str(bundle), norm_fn)
    norm = NormalizationData(norm_fn)
    all_x = numpy.concatenate([v[0] for v in ref.values()])
    assert numpy.allclose(norm.inputMean, all_x.mean(axis=0)) and numpy.allclose(norm.inputVariance, all_x.var(axis=0))
    ds = StereoHdfDataset(str(bundle), normalizationFile=norm_fn)
    ds.initialize()
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 6 and ds.num_inputs == 3 and ds.num_outputs["classes"] == (2, 2)
    got = []
    for i in range(6):
        ds.load_seqs(i, i + 1)
        got.append(ds.get_data(i, "data"))
    stacked = numpy.concatenate(got)
    assert abs(stacked.mean()) < 1e-5 and abs(stacked.var(axis=0).mean() - 1.0) < 1e-4
    ctx = DatasetWithTimeContext(files[0], tau=2)
    ctx.initialize()
    ctx.init_seq_order(epoch=1)
    ctx.load_seqs(0, 1)
    x = ref[(0, 0)][0].astype("float32")
    out = ctx.get_data(0, "data")
    assert out.shape == (4, 15) and numpy.allclose(out[1, 6:9], x[1]) and numpy.allclose(out[0, 0:3], x[0]) and numpy.allclose(out[3, 12:15], x[3])
    with pytest.raises(ValueError):
        with h5py.File(str(tmp_path / "in_only.hdf"), "w") as f:
            f.create_group("inputs").create_dataset("0", data=numpy.zeros((3, 2)))
        StereoHdfDataset(str(tmp_path / "in_only.hdf"))


def test_raw_wav_dataset_frames(tmp_path):
    from returnn_b200.datasets.raw_wav import RawWavDataset

    sig = numpy.sin(numpy.arange(1000) * 0.05) * 0.5
    _write_wav(tmp_path / "a.wav", sig)
    _write_wav(tmp_path / "b.wav", sig[:330])
    lst = tmp_path / "wavs.lst"
    lst.write_text("%s\n%s\n" % (tmp_path / "a.wav", tmp_path / "b.wav"))
    ds = RawWavDataset(str(lst), frameLength=100, frameShift=50, num_outputs=1)
    ds.init_seq_order(epoch=1)
    ds.load_seqs(0, 2)
    a, b = ds.get_data(0, "data"), ds.get_data(1, "data")
    assert a.shape == (19, 100) and b.shape == (6, 100)
    assert numpy.allclose(a[1, :50], a[0, 50:]) and numpy.allclose(a[0], sig[:100], atol=1e-4)
    assert numpy.allclose(b[5, :80], sig[250:330], atol=1e-4) and float(numpy.abs(b[5, 80:]).max()) == 0.0
    with pytest.raises(ValueError):
        RawWavDataset(str(lst), frameLength=100, frameShift=50)


def test_librispeech_timit_bliss_enwik8_corpora(tmp_path):
    import zipfile
    from returnn_b200.datasets.generating import LibriSpeechCorpus, TimitDataset, BlissDataset, Enwik8Corpus

    rng = numpy.random.RandomState(2)
    # --- LibriSpeech tree (wav instead of flac: no decoder for flac here)
    root = tmp_path / "libri"
    for sub, speaker, chapter, n in (("train-clean-100", 19, 198, 3), ("train-other-500", 20, 205, 2), ("dev-clean", 84, 121, 2)):
        d = root / sub / str(speaker) / str(chapter)
        d.mkdir(parents=True)
        lines = []
        for i in range(n):
            _write_wav(d / ("%i-%i-%04i.wav" % (speaker, chapter, i)), rng.uniform(-0.3, 0.3, size=4000 + 800 * i))
            lines.append("%i-%i-%04i HELLO WORLD %s" % (speaker, chapter, i, "A" * i))
        (d / ("%i-%i.trans.txt" % (speaker, chapter))).write_text("\n".join(lines) + "\n")
    ds = LibriSpeechCorpus(str(root), prefix="train", audio={"features": "mfcc", "num_feature_filters": 13}, chars={"vocab_file": None, "labels": list(" ABCDEHLORW")}
                           if False else None, targets={"class": "Utf8ByteTargets"}, orth_post_process="lowercase", seq_ordering="sorted")
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 5 and ds.get_all_tags()[0] == "train-clean-100-19-198-0000"
    ds.load_seqs(0, 5)
    assert ds.get_data(0, "data").shape[1] == 13 and ds.get_data(0, "data").shape[0] > 10
    assert bytes(ds.get_data(4, "orth")).decode() == "hello world aa" and ds.get_data(0, "classes").dtype == numpy.int32
    # --- TIMIT
    troot = tmp_path / "timit" / "train" / "dr1" / "fcjf0"
    troot.mkdir(parents=True)
    for utt in ("sa1", "si1027", "sx37"):
        _write_wav(troot / (utt + ".wav"), rng.uniform(-0.3, 0.3, size=8000))
        (troot / (utt + ".phn")).write_text("0 2000 h#\n2000 5000 aa\n5000 6400 q\n6400 8000 ux\n")
    td = TimitDataset(str(tmp_path / "timit"), train=True, num_feature_filters=13, num_phones=39)
    td.init_seq_order(epoch=1)
    assert td.num_seqs == 2 and len(td.labels["classes"]) == 39
    td.load_seqs(0, 1)
    x, c = td.get_data(0, "data"), td.get_data(0, "classes")
    assert x.shape[0] == c.shape[0] and x.shape[1] == 13
    lab = td.labels["classes"]
    assert lab[c[2]] == "sil" and lab[c[20]] == "aa" and lab[c[45]] == "uw"
    # --- Bliss
    _write_wav(tmp_path / "rec1.wav", rng.uniform(-0.3, 0.3, size=16000))
    (tmp_path / "corpus.xml").write_text(
        '<?xml version="1.0"?><corpus name="demo"><recording name="rec1" audio="rec1.wav">'
        '<segment name="1" start="0.0" end="0.4"><orth> ab  ba </orth></segment><segment name="2" start="0.4" end="1.0"><orth>b</orth></segment>'
        "</recording></corpus>")
    (tmp_path / "vocab.txt").write_text(repr({"ab": 0, "ba": 1, "b": 2}))
    bd = BlissDataset(str(tmp_path / "corpus.xml"), vocab_file=str(tmp_path / "vocab.txt"), num_feature_filters=13)
    bd.init_seq_order(epoch=1)
    bd.load_seqs(0, 2)
    assert bd.get_tag(0) == "demo/rec1/1" and bd.get_data(0, "classes").tolist() == [0, 1] and bd.get_data(1, "classes").tolist() == [2]
    assert bd.get_data(1, "data").shape[0] > bd.get_data(0, "data").shape[0]
    # --- enwik8
    edir = tmp_path / "enwik8"
    edir.mkdir()
    text = bytes(rng.randint(97, 105, size=5000).astype("uint8"))
    with zipfile.ZipFile(str(edir / "enwik8.zip"), "w") as z:
        z.writestr("enwik8", text)
    ed = Enwik8Corpus(str(edir), subset="training", seq_len=50, batch_num_seqs=4)
    ed.init_seq_order(epoch=1)
    n = ed.num_seqs
    assert n % 4 == 0 and n == (4000 // 50 // 4) * 4
    ed.load_seqs(0, 8)
    d0, c0 = ed.get_data(0, "data"), ed.get_data(0, "classes")
    assert d0.shape == (50,) and numpy.array_equal(d0[1:], c0[:-1]) and ed.get_tag(0) == "offset_0_50"
    # batch entry 0 of the next batch continues where entry 0 of this batch stopped
    assert ed.get_tag(4) == "offset_50_50" and ed.get_tag(1) == "offset_%i_50" % (50 * (n // 4))


def test_huggingface_dataset_wrapper():
    import datasets
    from returnn_b200.datasets.huggingface import HuggingFaceDataset

    hf = datasets.Dataset.from_dict({"id": ["u%i" % i for i in range(6)], "text": ["ab", "a", "bba", "abab", "b", "aab"],
                                     "feat": [numpy.arange(2 * (i + 1), dtype="float32").reshape(i + 1, 2).tolist() for i in range(6)],
                                     "n": [2, 1, 3, 4, 1, 3]})
    ds = HuggingFaceDataset(lambda: hf, data_format={"text": {"vocab": {"class": "CharacterTargets", "vocab_file": None, "labels": ["a", "b"], "unknown_label": None}},
                                                     "feat": {"dim": 2, "ndim": 2}},
                            sorting_seq_len_column="n", seq_ordering="sorted")
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 6 and ds.get_data_dim("text") == 2 and ds.is_data_sparse("text") and not ds.is_data_sparse("feat")
    lens = []
    for i in range(6):
        ds.load_seqs(i, i + 1)
        t = ds.get_data(i, "text")
        lens.append(len(t))
        corpus_idx = ds.get_corpus_seq_idx(i)
        assert ds.get_tag(i) == "u%i" % corpus_idx and ds.get_data(i, "feat").shape == (corpus_idx + 1, 2)
    assert lens == sorted(lens)


def _pp_scale(td, *, epoch, seq_idx, rng, **_):
    td.data["data"].raw_tensor = td.data["data"].raw_tensor * 2.0 + seq_idx
    return td


def _pp_drop_every_third(it, *, epoch, rng, **_):
    for i, td in enumerate(it):
        if i % 3 != 2:
            yield td


def test_postprocessing_dataset_worker_processes():
    """the same sequences, in the same order, with and without worker processes; functions may come from a config (by value)"""
    from returnn_b200.datasets.basic import init_dataset

    sub = {"class": "DummyDataset", "input_dim": 3, "output_dim": 4, "num_seqs": 11, "seq_len": 6}

    def read(ds, epoch):
        ds.init_seq_order(epoch=epoch)
        out, i = [], 0
        while ds.is_less_than_num_seqs(i):
            ds.load_seqs(i, i + 1)
            out.append((ds.get_tag(i), ds.get_data(i, "data").copy(), ds.get_data(i, "classes").copy()))
            i += 1
        return out

    plain = init_dataset({"class": "PostprocessingDataset", "dataset": sub, "map_seq": _pp_scale})
    multi = init_dataset({"class": "PostprocessingDataset", "dataset": sub, "map_seq": _pp_scale, "num_workers": 2, "buf_size": 3})
    try:
        for epoch in (1, 2):
            a, b = read(plain, epoch), read(multi, epoch)
            assert len(a) == len(b) == 11
            for (ta, xa, ca), (tb, xb, cb) in zip(a, b):
                assert ta == tb and numpy.array_equal(xa, xb) and numpy.array_equal(ca, cb)
    finally:
        multi.finish_epoch(free_resources=True)
    # a stream function per worker: every worker drops each third sequence of ITS share; functions defined in an exec'd config
    cfg = {"__name__": "__returnn_config__"}
    exec("def drop(it, *, epoch, rng, **_):\n    for i, td in enumerate(it):\n        if i % 3 != 2:\n            yield td\n", cfg)
    stream = init_dataset({"class": "PostprocessingDataset", "dataset": sub, "map_seq_stream": cfg["drop"], "num_workers": 2})
    try:
        tags = [t for t, _, _ in read(stream, 1)]
        # worker 0 has seqs 0,2,4,6,8,10 and drops its 3rd and 6th (4, 10); worker 1 has 1,3,5,7,9 and drops 5
        assert tags == ["seq-%i" % i for i in (0, 1, 2, 3, 6, 7, 8, 9)], tags
        assert stream.num_seqs == 8
    finally:
        stream.finish_epoch(free_resources=True)


def test_cached_dataset_budget_eviction_and_accessors():
    from returnn_b200.datasets.cached import CachedDataset

    class Ten(CachedDataset):
        def __init__(self, **kw):
            super().__init__(**kw)
            self._seq_tags = ["s%i" % i for i in range(10)]
            self._seq_lengths = numpy.array([[3 + i, 1] for i in range(10)])
            self._keys = ["data", "classes"]
            self.num_inputs = 2
            self.num_outputs = {"data": (2, 2), "classes": (5, 1)}
            self.loads = []

        def _load_seq_data(self, ci):
            self.loads.append(ci)
            return {"data": numpy.full((3 + ci, 2), ci, dtype="float32"), "classes": numpy.array([ci % 5], dtype="int32")}

    per_seq = lambda i: (3 + i) * 2 * 4 + 4
    ds = Ten(cache_byte_size=per_seq(0) + per_seq(1) + per_seq(2) + 8)
    ds.initialize()
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 10 and ds.get_seq_start(3).tolist() == [3 + 4 + 5, 3] and ds.get_seq_length_nd(2).tolist() == [5, 1]
    ds.load_seqs(0, 3)
    assert ds.is_cached(0, 3) and ds.loads == [0, 1, 2]
    ds.load_seqs(3, 4)  # needs room: the least recently used sequences leave
    assert not ds.is_cached(0, 1) and ds.is_cached(3, 4)
    assert ds.get_data(3, "data").shape == (6, 2) and ds.get_corpus_seq_idx(3) == 3 and ds.get_tag(3) == "s3"
    freed = ds.delete(1)
    assert freed >= 1 and ds._cache_bytes >= 0
    assert not ds.batch_set_generator_cache_whole_epoch()


def _write_translation_fixture(tmp_path, source_lines, target_lines, extra_vocabs=None):
    import pickle

    def vocab(words):
        return {w: i for i, w in enumerate(sorted(set(words)))}

    (tmp_path / "source.train").write_text("\n".join(source_lines) + "\n")
    (tmp_path / "target.train").write_text("\n".join(target_lines) + "\n")
    for name, v in (extra_vocabs or {}).items():
        with open(tmp_path / ("%s.vocab.pkl" % name), "wb") as f:
            pickle.dump(v, f)
    return vocab


def test_translation_factors_dataset(tmp_path):
    from returnn_b200.datasets.basic import init_dataset

    src = ["this|u is|l an|l example|u", "short|l"]
    tgt = ["das|u|x ist|l|y", "kurz|l|x"]
    _write_translation_fixture(tmp_path, src, tgt, extra_vocabs={
        "source": {"this": 0, "is": 1, "an": 2, "example": 3, "short": 4, "</s>": 5}, "src_case": {"u": 0, "l": 1, "</s>": 2},
        "target": {"das": 0, "ist": 1, "kurz": 2, "</s>": 3}, "tgt_case": {"u": 0, "l": 1, "</s>": 2}, "tgt_tag": {"x": 0, "y": 1, "</s>": 2}})
    ds = init_dataset({"class": "TranslationFactorsDataset", "path": str(tmp_path), "file_postfix": "train", "source_factors": "src_case",
                       "target_factors": ["tgt_case", "tgt_tag"], "source_postfix": " </s>", "target_postfix": " </s>"})
    ds.init_seq_order(epoch=1)
    assert ds.get_data_keys() == ["data", "src_case", "classes", "tgt_case", "tgt_tag"] and ds.get_target_list() == ["classes", "tgt_case", "tgt_tag"]
    ds.load_seqs(0, 2)
    assert ds.get_data(0, "data").tolist() == [0, 1, 2, 3, 5] and ds.get_data(0, "src_case").tolist() == [0, 1, 1, 0, 2]
    assert ds.get_data(0, "classes").tolist() == [0, 1, 3] and ds.get_data(0, "tgt_case").tolist() == [0, 1, 2] and ds.get_data(0, "tgt_tag").tolist() == [0, 1, 2]
    assert ds.get_data(1, "tgt_tag").tolist() == [0, 2] and ds.get_data_dim("tgt_tag") == 3


def test_confusion_network_dataset(tmp_path):
    from returnn_b200.datasets.basic import init_dataset

    src = ["__ALT__ we're|0.75__were|0.25 a|0.9__EPS|0.1 species|1.0", "plain text here"]
    tgt = ["x y", "z"]
    _write_translation_fixture(tmp_path, src, tgt, extra_vocabs={
        "source": {"PAD": 0, "we're": 1, "were": 2, "a": 3, "EPS": 4, "species": 5, "UNK": 6}, "target": {"x": 0, "y": 1, "z": 2}})
    ds = init_dataset({"class": "ConfusionNetworkDataset", "path": str(tmp_path), "file_postfix": "train", "max_density": 3, "unknown_label": {"data": "UNK"}})
    ds.init_seq_order(epoch=1)
    ds.load_seqs(0, 2)
    assert ds.get_data_keys() == ["sparse_inputs", "sparse_weights", "classes"]
    ids, w = ds.get_data(0, "sparse_inputs"), ds.get_data(0, "sparse_weights")
    assert ids.tolist() == [[1, 2, 0], [3, 4, 0], [5, 0, 0]] and w.dtype == numpy.float32
    numpy.testing.assert_allclose(w, [[0.75, 0.25, 0], [0.9, 0.1, 0], [1, 0, 0]])
    assert ds.get_data(1, "sparse_inputs")[:, 0].tolist() == [6, 6, 6] and ds.get_data(1, "sparse_weights")[:, 0].tolist() == [1.0, 1.0, 1.0]
    assert ds.get_data(1, "classes").tolist() == [2] and ds.get_data_shape("sparse_weights") == [3] and not ds.is_data_sparse("sparse_inputs")


def test_allophone_state_and_state_tying(tmp_path):
    from returnn_b200.datasets.lm import AllophoneState, StateTying

    phones = {"a": 0, "b": 1, "sil": 2}
    a = AllophoneState("a", 1)
    a.context_history, a.context_future = ("b",), ("sil",)
    a.mark_initial()
    assert a.format() == "a{b+sil}@i.1"
    idx = a.index(phones, num_states=3, context_length=1)
    back = AllophoneState.from_index(idx, {v: k for k, v in phones.items()}, num_states=3, context_length=1)
    assert back == a and hash(back) == hash(a) and back.format() == a.format()
    seen = set()
    for c in phones:
        for st in range(3):
            x = AllophoneState(c, st)
            seen.add(x.index(phones))
    assert len(seen) == 9
    f = tmp_path / "state-tying.txt"
    f.write_text("a{#+#}@i@f.0 0\na{#+#}@i@f.1 1\nb{a+#}.0 0\n# comment\n")
    t = StateTying(str(f))
    assert t.num_classes == 2 and t.allo_map["b{a+#}.0"] == 0 and t.class_map[0] == {"a{#+#}@i@f.0", "b{a+#}.0"}


def test_nltk_timit_layout_and_sequential_postprocessing(tmp_path):
    from returnn_b200.datasets.generating import NltkTimitDataset
    from returnn_b200.datasets.postprocessing import Sequential

    rng = numpy.random.RandomState(3)
    root = tmp_path / "nltk_data" / "corpora" / "timit"
    for spk in ("dr1-fvmh0", "dr2-marc0"):
        d = root / spk
        d.mkdir(parents=True)
        for utt in ("sa1", "sa2", "si1466", "sx116", "sx206"):
            _write_wav(d / (utt + ".wav"), rng.uniform(-0.3, 0.3, size=6000))
            (d / (utt + ".phn")).write_text("0 1500 h#\n1500 4000 iy\n4000 6000 h#\n")
    train = NltkTimitDataset(nltk_download_dir=str(tmp_path / "nltk_data"), train=True, num_feature_filters=13)
    dev = NltkTimitDataset(nltk_download_dir=str(tmp_path / "nltk_data"), train=False, num_feature_filters=13)
    train.init_seq_order(epoch=1)
    dev.init_seq_order(epoch=1)
    assert train.num_seqs == 9 and dev.num_seqs == 1 and dev.get_all_tags() == ["dr2-marc0/sx206"]
    train.load_seqs(0, 1)
    c = train.get_data(0, "classes")
    assert train.labels["classes"][c[len(c) // 2]] == "iy"
    with pytest.raises(FileNotFoundError):
        NltkTimitDataset(nltk_download_dir=str(tmp_path / "nowhere"))

    def double(t, **kw):
        return t * 2

    def add_epoch(t, *, epoch=0, **kw):
        return t + epoch

    double.preserves_num_seqs = True
    seq = Sequential(double, add_epoch)
    assert seq(3, epoch=5) == 11 and not seq.preserves_num_seqs
    add_epoch.preserves_num_seqs = True
    assert Sequential(double, add_epoch).preserves_num_seqs


def test_batch_to_raw_dict_and_small_dataset_helpers():
    import io
    import logging
    import sys
    from returnn_b200.engine.batch import Batch, batch_to_raw_dict
    from returnn_b200.datasets.basic import init_dataset, extend_dataset_dict_from_parent_dataset
    from returnn_b200.datasets.util.strings import str_to_numpy_array
    from returnn_b200.torch.data.returnn_dataset_wrapper import ReturnnDatasetFullMapDataPipe
    from returnn_b200.pretrain import WrapEpochValue
    from returnn_b200.log import StdoutHandler, StreamDummy

    seqs = [{"data": numpy.arange(10, dtype="float32").reshape(5, 2), "classes": numpy.array([1, 2, 3], dtype="int32")},
            {"data": numpy.ones((2, 2), dtype="float32"), "classes": numpy.array([4], dtype="int32")}]
    ds = init_dataset({"class": "StaticDataset", "data": seqs, "output_dim": {"data": (2, 2), "classes": (5, 1)}})
    ds.init_seq_order(epoch=1)
    b = Batch()
    from returnn_b200.utils.basic import NumbersDict as ND

    b.add_sequence_as_slice(0, ND({"data": 1, "classes": 0}), ND({"data": 3, "classes": 3}))  # a chunk of sequence 0
    b.add_sequence_as_slice(1, ND({"data": 0, "classes": 0}), ND({"data": 2, "classes": 1}))
    raw = batch_to_raw_dict(b, dataset=ds, data_keys=["data", "classes"])
    assert raw["data"].shape == (2, 3, 2) and raw["data"][0].tolist() == [[2, 3], [4, 5], [6, 7]] and raw["data"][1, 2].tolist() == [0, 0]
    assert raw["data_seq_lens"].tolist() == [3, 2] and raw["classes_seq_lens"].tolist() == [3, 1] and raw["classes"][1].tolist() == [4, 0, 0]
    assert raw["seq_idx"].tolist() == [0, 1] and int(raw["batch_dim"]) == 2 and len(raw["seq_tag"]) == 2
    fw = Batch()
    fw.add_frames(0, ND({"data": 0, "classes": 0}), ND({"data": 5, "classes": 3}))
    fw.add_frames(1, ND({"data": 0, "classes": 0}), ND({"data": 2, "classes": 1}))
    raw2 = batch_to_raw_dict(fw, dataset=ds, data_keys=["data"])
    assert raw2["data"].shape == (1, 7, 2) and raw2["data_seq_lens"].tolist() == [7] and raw2["data"][0, 5].tolist() == [1, 1]
    parent = init_dataset({"class": "StaticDataset", "data": seqs, "output_dim": {"data": (2, 2), "classes": (5, 1)}, "random_seed_offset": 77})
    assert extend_dataset_dict_from_parent_dataset({"class": "X"}, parent) == {"class": "X", "random_seed_offset": 77}
    assert extend_dataset_dict_from_parent_dataset({"class": "X", "random_seed_offset": 1}, parent)["random_seed_offset"] == 1
    assert str_to_numpy_array("abc").dtype.kind == "U" and str_to_numpy_array("abc").shape == ()
    pipe = ReturnnDatasetFullMapDataPipe(ds)
    assert len(pipe) == 2 and pipe[1]["classes"].tolist() == [4]
    assert WrapEpochValue(lambda epoch: epoch * 2).get_value(3) == 6
    buf = io.StringIO()
    old = sys.stdout
    try:
        h = StdoutHandler()
        sys.stdout = buf
        logging.Logger("t").handle  # noqa: B018
        h.emit(logging.LogRecord("t", logging.INFO, __file__, 1, "hello %s", ("x",), None))
    finally:
        sys.stdout = old
    assert "hello x" in buf.getvalue()
    StreamDummy().write("ignored")
