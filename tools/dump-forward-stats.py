#!/usr/bin/env python3
"""
Mean and standard deviation per feature of a model output over a dataset (e.g. to normalise an intermediate representation).
Writes ``<prefix>.mean.txt`` and ``<prefix>.std_dev.txt``. (reference: tools/dump-forward-stats.py)
"""

import argparse
import numpy
import _setup_returnn_env  # noqa: F401
from returnn_b200 import __main__ as rnn
from returnn_b200.forward_iface import ForwardCallbackIface


class _Stats(ForwardCallbackIface):
    def __init__(self, key):
        self.key = key
        self.n = 0
        self.s1 = None
        self.s2 = None

    def process_seq(self, *, seq_tag, outputs):
        out = outputs[self.key]
        arr = out.raw_tensor.double().numpy() if hasattr(out.raw_tensor, "numpy") else numpy.asarray(out.raw_tensor, dtype="float64")
        axis = out.feature_dim_axis if out.feature_dim_axis is not None else arr.ndim - 1
        arr = numpy.moveaxis(arr, axis, -1).reshape(-1, arr.shape[axis])
        self.n += arr.shape[0]
        self.s1 = arr.sum(0) if self.s1 is None else self.s1 + arr.sum(0)
        self.s2 = (arr ** 2).sum(0) if self.s2 is None else self.s2 + (arr ** 2).sum(0)


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config")
    ap.add_argument("--epoch", type=int, default=None)
    ap.add_argument("--data", default="train")
    ap.add_argument("--output-key", default="output")
    ap.add_argument("--prefix", default="stats")
    args, rest = ap.parse_known_args()
    opts = ["++task", "forward", "++log_verbosity", "3", "++allow_skipping_seqs_in_forward", "True"]
    if args.epoch is not None:
        opts += ["++load_epoch", str(args.epoch)]
    cb = _Stats(args.output_key)
    rnn.init(config_filename=args.config, command_line_options=opts + rest, config_updates={"forward_callback": cb, "forward_data": eval(args.data) if args.data.strip().startswith("{") else args.data})
    try:
        rnn.execute_main_task()
    finally:
        rnn.finalize()
    mean = cb.s1 / cb.n
    std = numpy.sqrt(numpy.maximum(cb.s2 / cb.n - mean ** 2, 0.0))
    numpy.savetxt(args.prefix + ".mean.txt", mean)
    numpy.savetxt(args.prefix + ".std_dev.txt", std)
    print("%i frames, %i features -> %s.{mean,std_dev}.txt" % (cb.n, len(mean), args.prefix))


if __name__ == "__main__":
    main()
