#!/usr/bin/env python3
"""
A stand-in for an embedding RASR process: it calls the entry points of ``returnn_b200.sprint.extern_interface`` the way RASR's Python
trainer does (``getSegmentList``, ``init``, ``feedInputAndTargetAlignment`` per segment, ``exit``). Run it directly to see the dataset
side, or give it as ``sprintTrainerExecPath`` of an ``ExternSprintDataset``:

    python demos/demo-sprint-interface.py

starts itself once more as the producer child and prints the sequences that arrive through the pipe.
"""

import sys
import _setup_env  # noqa: F401
import numpy


def producer(argv):
    """the child side: options as ExternSprintDataset appends them (``--*.key=value``)"""
    import importlib

    opts = {}
    for a in argv:
        if a.startswith("--*."):
            k, _, v = a[4:].partition("=")
            opts[k] = v
    sys.path.insert(0, opts["pymod-path"])
    mod = importlib.import_module(opts["pymod-name"])
    rng = numpy.random.RandomState(int(opts.get("seed", "1")))
    segments = ["demo-corpus/recording-%i/1" % i for i in range(int(opts.get("num-segments", "5")))]
    part, sel = int(opts.get("corpus.partition", "1")), int(opts.get("corpus.select-partition", "0"))
    segments = list(mod.getSegmentList("demo-corpus", segments[sel::part]))
    mod.init(inputDim=9, outputDim=2, config=opts["pymod-config"], targetMode="criterion-by-sprint")
    for name in segments:
        t = int(rng.randint(5, 12))
        mod.feedInputAndTargetAlignment(rng.randn(9, t).astype("float32"), rng.randint(0, 2, size=(t,)).astype("int32"), segmentName=name)
    mod.exit()


def main():
    if any(a.startswith("--*.pymod-name=") for a in sys.argv[1:]):
        producer(sys.argv[1:])
        return
    from returnn_b200.datasets.basic import init_dataset

    ds = init_dataset({"class": "ExternSprintDataset", "sprintTrainerExecPath": [sys.executable, __file__], "sprintConfigStr": "--*.num-segments=5"})
    print("dimensions announced by the producer:", ds.num_outputs)
    for epoch in (1, 2):
        ds.init_seq_order(epoch=epoch)
        i = 0
        while ds.is_less_than_num_seqs(i):
            ds.load_seqs(i, i + 1)
            print("epoch %i seq %i %s data %s classes %s" % (epoch, i, ds.get_tag(i), ds.get_data(i, "data").shape, ds.get_data(i, "classes").tolist()))
            i += 1
        ds.finish_epoch()


if __name__ == "__main__":
    main()
