#!/usr/bin/env python3
"""
Run ``forward_step`` of a config over a dataset and dump the outputs per sequence to an ``.npz`` archive (keys
``<seq_tag>/<output name>``) or print summaries.

    tools/dump-forward.py my.config --epoch 10 --data dev [--output out.npz] [--num-seqs 20]

(reference: tools/dump-forward.py, which writes HDF through the TF engine)
"""

import argparse
import numpy
import _setup_returnn_env  # noqa: F401
from returnn_b200 import __main__ as rnn
from returnn_b200.forward_iface import ForwardCallbackIface


class _Collect(ForwardCallbackIface):
    def __init__(self, limit):
        self.limit = limit
        self.data = {}
        self.n = 0

    def process_seq(self, *, seq_tag, outputs):
        if self.limit and self.n >= self.limit:
            return
        self.n += 1
        for k, v in outputs.data.items():
            raw = v.raw_tensor
            arr = raw.float().numpy() if hasattr(raw, "numpy") else numpy.asarray(raw)
            self.data["%s/%s" % (seq_tag, k)] = arr
            print("%s %s: shape %s mean %.5g" % (seq_tag, k, arr.shape, float(arr.mean()) if arr.size and arr.dtype.kind == "f" else 0.0))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config")
    ap.add_argument("--epoch", type=int, default=None, help="checkpoint epoch (default: config load / latest)")
    ap.add_argument("--data", default="dev", help="train, dev, eval or a dataset dict")
    ap.add_argument("--output", default=None)
    ap.add_argument("--num-seqs", type=int, default=0)
    ap.add_argument("--device", default=None)
    args, rest = ap.parse_known_args()
    opts = ["++task", "forward", "++log_verbosity", "3"]
    if args.epoch is not None:
        opts += ["++load_epoch", str(args.epoch)]
    if args.device:
        opts += ["++device", args.device]
    cb = _Collect(args.num_seqs)
    rnn.init(config_filename=args.config, command_line_options=opts + rest, config_updates={"forward_callback": cb, "forward_data": eval(args.data) if args.data.strip().startswith("{") else args.data})
    try:
        rnn.execute_main_task()
    finally:
        rnn.finalize()
    if args.output:
        numpy.savez_compressed(args.output, **cb.data)
        print("wrote %i arrays to %s" % (len(cb.data), args.output))


if __name__ == "__main__":
    main()
