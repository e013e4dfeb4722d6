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
