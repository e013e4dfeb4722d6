"""Producer-fed datasets: a thread pushing into SprintDatasetBase, and ExternSprintDataset with a stand-in producer process that speaks the pipe protocol
through returnn_b200.sprint.extern_interface exactly as an embedding RASR process would call it."""

import os
import sys
import textwrap
import threading
import numpy
import pytest


def test_sprint_dataset_base_producer_thread_and_back_pressure():
    from returnn_b200.datasets.sprint import SprintDatasetBase

    class Small(SprintDatasetBase):
        SprintCachedSeqsMax = 6
        SprintCachedSeqsMin = 3

    ds = Small(target_maps={"speaker_name": {"anna": 0, "bob": 1}}, str_add_final_zero=True, input_stddev=2.0, reduce_target_factor=2)
    ds.set_dimensions(3, 5)
    rng = numpy.random.RandomState(0)
    feats = [rng.randn(3, 4 + i).astype("float32") for i in range(20)]
    pushed = []

    def producer():
        ds.init_sprint_epoch(1)
        for i, f in enumerate(feats):
            t = f.shape[1]
            idx = ds.add_new_data(f.copy(), {"classes": numpy.arange((t + 1) // 2, dtype="int32") % 5, "orth": " hello %i " % i,
                                             "speaker_name": "bob" if i % 2 else "anna"}, segment_name="seg-%i" % i)
            pushed.append(idx)
        ds.finish_sprint_epoch()

    th = threading.Thread(target=producer, daemon=True)
    th.start()
    ds.init_seq_order(epoch=1)
    import time

    time.sleep(0.3)
    assert 6 <= len(pushed) <= 7  # held back at the high mark until the consumer asks for more
    i = 0
    while ds.is_less_than_num_seqs(i):
        ds.load_seqs(i, i + 1)
        x = ds.get_data(i, "data")
        numpy.testing.assert_allclose(x, feats[i].T / 2.0, rtol=1e-6)
        assert ds.get_tag(i) == "seg-%i" % i
        assert ds.get_data(i, "classes").shape == ((x.shape[0] + 1) // 2,)
        assert bytes(ds.get_data(i, "orth")).decode() == "hello %i" % i
        assert ds.get_data(i, "orth0")[-1] == 0
        spk = ds.get_data(i, "speaker_name")
        assert spk.shape == (x.shape[0],) and int(spk[0]) == i % 2
        assert ds.get_seq_length(i)["data"] == x.shape[0]
        i += 1
    th.join(5)
    assert i == 20 and ds.num_seqs == 20 and ds.get_num_timesteps() == sum(f.shape[1] for f in feats)
    assert ds.get_complete_frac(19) == 1.0
    assert set(ds.get_data_keys()) >= {"data", "classes", "orth", "orth0", "speaker_name"}


def test_sprint_dataset_base_checks_predefined_order_and_window():
    from returnn_b200.datasets.sprint import SprintDatasetBase

    ds = SprintDatasetBase(window=3)
    ds.set_dimensions(2, 0)
    ds.init_sprint_epoch(1)
    ds.init_seq_order(epoch=1, seq_list=["a", "b"])
    x = numpy.arange(8, dtype="float32").reshape(2, 4)
    ds.add_new_data(x, segment_name="a")
    got = ds.get_data(0, "data")
    assert got.shape == (4, 6)
    numpy.testing.assert_array_equal(got[0], [0, 0, 0, 4, 1, 5])  # zeros, frame 0, frame 1
    numpy.testing.assert_array_equal(got[3], [2, 6, 3, 7, 0, 0])
    with pytest.raises(Exception, match="should be 'b'"):
        ds.add_new_data(x, segment_name="c")
    assert ds.num_seqs == 2


_PRODUCER = textwrap.dedent('''
    """stand-in for an embedding RASR process: parses the options ExternSprintDataset appends and calls the module's entry points"""
    import sys, importlib
    import numpy
    opts = {}
    for a in sys.argv[1:]:
        if a.startswith("--*."):
            k, _, v = a[4:].partition("=")
            opts[k] = v
    sys.path.insert(0, opts["pymod-path"])
    mod = importlib.import_module(opts["pymod-name"])
    n = int(opts.get("num-seqs", "7"))
    segs = ["corpus/rec/%i" % i for i in range(n)]
    if "corpus.segments.file" in opts:
        segs = open(opts["corpus.segments.file"]).read().split()
    part, sel = int(opts.get("corpus.partition", "1")), int(opts.get("corpus.select-partition", "0"))
    segs = segs[sel::part]
    segs = list(mod.getSegmentList("corpus", segs))
    if opts.get("mode") == "control":
        ctl = mod.init(name="x", sprint_unit="u", config=opts["pymod-config"])
        ctl.init_processing(input_dim=4, output_dim=9)
        for s in segs:
            i = int(s.rsplit("/", 1)[1])
            ctl.process_segment(name=s, orthography="w%i" % i, features=numpy.full((4, 3 + i), float(i), dtype="float32"),
                                alignment=numpy.full((3 + i,), i % 9, dtype="int32"), soft_alignment=None)
        ctl.exit()
    else:
        mod.init(inputDim=4, outputDim=9, config=opts["pymod-config"], targetMode="criterion-by-sprint")
        for s in segs:
            i = int(s.rsplit("/", 1)[1])
            mod.feedInputAndTargetAlignment(numpy.full((4, 3 + i), float(i), dtype="float32"), numpy.full((3 + i,), i % 9, dtype="int32"), segmentName=s)
        mod.exit()
''')


@pytest.mark.parametrize("mode", ["trainer", "control"])
def test_extern_sprint_dataset_child_process(tmp_path, mode):
    from returnn_b200.datasets.basic import init_dataset

    script = tmp_path / "producer.py"
    script.write_text(_PRODUCER)
    ds = init_dataset({"class": "ExternSprintDataset", "sprintTrainerExecPath": [sys.executable, str(script)],
                       "sprintConfigStr": "--*.num-seqs=7 --*.mode=%s" % mode, "partition_epoch": 2})
    assert ds.num_inputs == 4 and ds.num_outputs["classes"] == (9, 1)
    seen = {}
    for epoch in (1, 2):
        ds.init_seq_order(epoch=epoch)
        i = 0
        tags = []
        while ds.is_less_than_num_seqs(i):
            ds.load_seqs(i, i + 1)
            tag = ds.get_tag(i)
            k = int(tag.rsplit("/", 1)[1])
            x = ds.get_data(i, "data")
            assert x.shape == (3 + k, 4) and float(x[0, 0]) == float(k)
            assert ds.get_data(i, "classes").tolist() == [k % 9] * (3 + k)
            if mode == "control":
                assert bytes(ds.get_data(i, "orth")).decode() == "w%i" % k
            tags.append(tag)
            i += 1
        assert ds.num_seqs == len(tags)
        seen[epoch] = tags
        ds.finish_epoch()
    assert seen[1] == ["corpus/rec/%i" % i for i in (0, 2, 4, 6)] and seen[2] == ["corpus/rec/%i" % i for i in (1, 3, 5)]
    # an explicit list of tags is handed to the producer as a segment file and checked on arrival
    ds2 = init_dataset({"class": "ExternSprintDataset", "sprintTrainerExecPath": [sys.executable, str(script)], "sprintConfigStr": ["--*.num-seqs=7"]})
    ds2.init_seq_order(epoch=1, seq_list=["corpus/rec/5", "corpus/rec/1"])
    assert ds2.num_seqs == 2
    ds2.load_seqs(0, 2)
    assert [ds2.get_tag(0), ds2.get_tag(1)] == ["corpus/rec/5", "corpus/rec/1"] and ds2.get_data(1, "data").shape == (4, 4)
    ds2.finish_epoch()


# ---- archive files (reader / writer) and the dataset over them ----


def _allophone_files(tmp_path):
    allos = ["si{#+#}@i@f", "a{#+b}@i", "b{a+#}@f", "a{b+a}"]
    (tmp_path / "allophones").write_text("# comment\n" + "\n".join(allos) + "\n")
    tying = {}
    for i, a in enumerate(allos):
        for s in range(3 if i else 1):
            tying["%s.%i" % (a, s)] = len(tying)
    (tmp_path / "state-tying").write_text("".join("%s %i\n" % kv for kv in tying.items()))
    (tmp_path / "phonemes").write_text("si\na\nb\n")
    return allos, tying


def _write_archives(tmp_path, n_seqs=5, dim=7, compress=False, seed=3):
    import numpy
    from returnn_b200.sprint.cache import FileArchive

    rnd = numpy.random.RandomState(seed)
    allos, tying = _allophone_files(tmp_path)
    feats, aligns = {}, {}
    fa = FileArchive(str(tmp_path / "feat.cache"), must_exists=False)
    aa = FileArchive(str(tmp_path / "align.cache"), must_exists=False)
    for i in range(n_seqs):
        name = "corpus/rec%i/seg%i" % (i // 2, i)
        T = int(rnd.randint(5, 40))
        x = rnd.randn(T, dim).astype("float32")
        times = [(0.01 * t, 0.01 * (t + 1)) for t in range(T)]
        fa.add_feature_cache(name, x, times, compress=compress)
        # runs of one allophone state, some single frames in between (both forms of the run-length code)
        em = []
        while len(em) < T:
            a = int(rnd.randint(0, len(allos)))
            s = int(rnd.randint(0, 3)) if a else 0
            em += [a + (s << 26)] * int(rnd.choice([1, 1, 2, 5]))
        em = em[:T]
        aa.add_alignment(name, em, compress=compress)
        feats[name], aligns[name] = x, em
    fa.finalize()
    aa.finalize()
    return feats, aligns, allos, tying


import pytest


@pytest.mark.parametrize("compress", [False, True])
def test_archive_round_trip(tmp_path, compress):
    import numpy
    from returnn_b200.sprint import cache

    feats, aligns, allos, tying = _write_archives(tmp_path, compress=compress)
    assert cache.is_sprint_cache_file(str(tmp_path / "feat.cache")) and not cache.is_sprint_cache_file(str(tmp_path / "phonemes"))
    arc = cache.open_file_archive(str(tmp_path / "feat.cache"))
    assert sorted(n for n in arc.file_list() if not n.endswith(".attribs")) == sorted(feats)
    for name, x in feats.items():
        times, rows = arc.read(name, "feat")
        numpy.testing.assert_array_equal(numpy.asarray(rows), x)
        assert abs(times[-1][1] - 0.01 * len(x)) < 1e-9
        assert arc.read(os.path.basename(name), "feat")[1][0].shape == (x.shape[1],)  # lookup by the unique base name
        assert 'name="sample-size" value="%i"' % x.shape[1] in arc.read(name + ".attribs", "str")
    al = cache.open_file_archive(str(tmp_path / "align.cache"))
    al.set_allophones(str(tmp_path / "allophones"))
    assert al.get_allophones_list() == allos
    for name, em in aligns.items():
        got = al.read(name, "align")
        assert [t for (t, _, _, _) in got] == list(range(len(em)))
        assert [a + (s << 26) for (_, a, s, _) in got] == em and all(w == 1 for (_, _, _, w) in got)
        assert [e for (_, e, _, _) in al.read(name, "align_raw")] == em


def test_archive_weighted_alignment_bundle_and_scan(tmp_path):
    import numpy
    from returnn_b200.sprint import cache

    allos, _ = _allophone_files(tmp_path)
    a1 = cache.FileArchive(str(tmp_path / "a1.cache"), must_exists=False)
    a1.add_alignment("s1", [1, 1 + (2 << 26), 300 % 4], weights=[0.5, 0.25, 1.0])
    a1.add_feature_cache("s1f", numpy.ones((3, 2), "float32"), [(0, 1), (1, 2), (2, 3)])
    a1.finalize()
    a2 = cache.FileArchive(str(tmp_path / "a2.cache"), must_exists=False)
    a2.add_feature_cache("s2f", numpy.zeros((2, 2), "float32"), [(0, 1), (1, 2)])
    a2.finalize()
    (tmp_path / "all.bundle").write_text("a1.cache\n%s\n" % (tmp_path / "a2.cache"))
    bundle = cache.open_file_archive(str(tmp_path / "all.bundle"))
    assert isinstance(bundle, cache.FileArchiveBundle) and bundle.has_entry("s2f") and bundle.has_entry("s1")
    bundle.set_allophones(str(tmp_path / "allophones"))
    assert bundle.read("s1", "align") == [(0, 1, 0, 0.5), (1, 1, 2, 0.25), (2, 0, 0, 1.0)]
    assert len(bundle.read("s2f", "feat")[1]) == 2
    # an archive without a table of contents is walked by its entry tags
    raw = bytearray(open(tmp_path / "a1.cache", "rb").read())
    raw[8] = 0
    open(tmp_path / "a1-no-toc.cache", "wb").write(bytes(raw))
    scanned = cache.FileArchive(str(tmp_path / "a1-no-toc.cache"))
    assert set(scanned.file_list()) == set(a1.ft) and len(scanned.read("s1f", "feat")[1]) == 3
    # the command line tool
    import io
    import contextlib

    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        cache.main([str(tmp_path / "a1.cache")])
        cache.main([str(tmp_path / "a1.cache"), "s1", "--mode", "show", "--type", "align", "--allophone-file", str(tmp_path / "allophones")])
    out = buf.getvalue()
    assert "s1f.attribs" in out and "allophone=a{#+b}@i\tindex=1\tstate=2\tweight=0.25" in out


def test_mixture_set_and_word_boundaries(tmp_path):
    import struct
    import numpy
    from returnn_b200.sprint.cache import MixtureSet, WordBoundaries

    ms = MixtureSet()
    ms.version, ms.dim = 2, 3
    ms.means, ms.mean_weights = numpy.arange(6.0).reshape(2, 3), numpy.array([1.0, 2.0])
    ms.covs, ms.cov_weights = numpy.ones((1, 3)) * 0.5, numpy.array([3.0])
    ms.densities = numpy.array([[0, 0], [1, 0]], dtype=numpy.int32)
    ms.mixtures = [([0], [1.0]), ([1, 0], [0.25, 0.75])]
    ms.write(str(tmp_path / "mix"))
    back = MixtureSet(str(tmp_path / "mix"))
    assert (back.version, back.dim, back.num_means, back.num_covs, back.num_densities, back.get_number_mixtures()) == (2, 3, 2, 1, 2, 2)
    numpy.testing.assert_array_equal(back.means, ms.means)
    numpy.testing.assert_array_equal(back.get_mean_by_idx(1), numpy.float32([3, 4, 5]))
    numpy.testing.assert_array_equal(back.get_cov_by_idx(0), numpy.float32([0.5] * 3))
    assert back.mixtures == ms.mixtures
    with open(tmp_path / "wb", "wb") as f:
        f.write(b"LATWRDBN" + struct.pack("<II", 1, 2) + struct.pack("<IHH", 10, 3, 4) + struct.pack("<IHH", 20, 5, 6))
    assert WordBoundaries(str(tmp_path / "wb")).boundaries == [(10, 4, 3), (20, 6, 5)]


@pytest.mark.parametrize("labels", ["state_tying", "phonemes"])
def test_sprint_cache_dataset(tmp_path, labels):
    import numpy
    from returnn_b200.datasets.basic import init_dataset

    feats, aligns, allos, tying = _write_archives(tmp_path, n_seqs=6)
    labeling = {"silence_phone": "si", "allophone_file": str(tmp_path / "allophones")}
    labeling["state_tying_file" if labels == "state_tying" else "phoneme_file"] = str(tmp_path / labels.replace("_", "-") if labels == "state_tying" else tmp_path / "phonemes")
    ds = init_dataset({"class": "SprintCacheDataset", "seq_ordering": "sorted", "data": {
        "data": {"filename": str(tmp_path / "feat.cache")}, "classes": {"filename": str(tmp_path / "align.cache"), "allophone_labeling": labeling}}})
    assert ds.num_inputs == 7 and ds.num_outputs["classes"] == (len(tying) if labels == "state_tying" else 3, 1)
    assert ds.get_target_list() == ["classes"] and sorted(ds.get_all_tags()) == sorted(feats)
    ds.init_seq_order(epoch=1)
    assert ds.num_seqs == 6
    lens = []
    for i in range(ds.num_seqs):
        ds.load_seqs(i, i + 1)
        tag = ds.get_tag(i)
        numpy.testing.assert_array_equal(ds.get_data(i, "data"), feats[tag])
        want = [tying["%s.%i" % (allos[e & ((1 << 26) - 1)], e >> 26)] if labels == "state_tying" else ["si", "a", "b"].index(allos[e & ((1 << 26) - 1)].split("{")[0])
                for e in aligns[tag]]
        assert ds.get_data(i, "classes").tolist() == want and ds.get_data(i, "classes").dtype == numpy.int8
        lens.append(len(feats[tag]))
    assert lens == sorted(lens)  # "sorted" works from the entry sizes in the table of contents


def test_archives_agree_with_the_reference_reader_and_writer(tmp_path):
    """an archive written here reads the same through the reference's reader, and one written by the reference reads the same here"""
    import numpy
    import _parity as P

    if not P.reference_available():
        pytest.skip("reference package not installed under baseline/_ref")
    P.reference()
    from returnn.sprint import cache as ref_cache
    from returnn_b200.sprint import cache

    feats, aligns, allos, _ = _write_archives(tmp_path, compress=True)
    rf_ = ref_cache.open_file_archive(str(tmp_path / "feat.cache"))
    ra = ref_cache.open_file_archive(str(tmp_path / "align.cache"))
    ra.set_allophones(str(tmp_path / "allophones"))
    mine = cache.open_file_archive(str(tmp_path / "align.cache"))
    mine.set_allophones(str(tmp_path / "allophones"))
    for name in feats:
        t_ref, x_ref = rf_.read(name, "feat")
        numpy.testing.assert_array_equal(numpy.asarray(x_ref), feats[name])
        assert [tuple(x) for x in ra.read(name, "align")] == [tuple(x) for x in mine.read(name, "align")]
    w = ref_cache.FileArchive(str(tmp_path / "ref.cache"), must_exists=False)
    x = numpy.random.RandomState(1).randn(9, 4).astype("float32")
    w.add_feature_cache("seq", x, [(float(t), float(t + 1)) for t in range(9)])
    w.finalize()
    w.f.close()
    times, rows = cache.FileArchive(str(tmp_path / "ref.cache")).read("seq", "feat")
    numpy.testing.assert_array_equal(numpy.asarray(rows), x)
    assert [tuple(t) for t in times] == [(float(t), float(t + 1)) for t in range(9)]
