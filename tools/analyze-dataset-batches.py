#!/usr/bin/env python3
"""
Batch statistics of a dataset under given batching options: number of batches, sequences per batch, padding ratio
(reference: tools/analyze-dataset-batches.py).

    tools/analyze-dataset-batches.py my.config --dataset train --batch_size 40000 --max_seqs 200
"""

import argparse
import sys
import _setup_returnn_env  # noqa: F401
from returnn_b200.config import Config
from returnn_b200.datasets.basic import init_dataset
from returnn_b200.torch.data import pipeline, returnn_dataset_wrapper


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config_or_dataset")
    ap.add_argument("--dataset", default="train")
    ap.add_argument("--epoch", type=int, default=1)
    ap.add_argument("--batch_size", type=int, default=None)
    ap.add_argument("--max_seqs", type=int, default=None)
    ap.add_argument("--key", default="data")
    args = ap.parse_args()
    text = args.config_or_dataset.strip()
    cfg = Config()
    if text.startswith("{"):
        ds_opts = eval(text)
    else:
        cfg.load_file(text)
        ds_opts = cfg.typed_value(args.dataset)
    batch_size = args.batch_size if args.batch_size is not None else cfg.typed_value("batch_size", 0)
    max_seqs = args.max_seqs if args.max_seqs is not None else cfg.int("max_seqs", -1)
    ds = init_dataset(ds_opts)
    wrapped = returnn_dataset_wrapper.ReturnnDatasetIterDataPipe(ds, reset_callback=lambda: ds.init_seq_order(epoch=args.epoch))
    batches = pipeline.BatchingIterDataPipe(wrapped, batch_size=batch_size, max_seqs=max_seqs)
    n_batches = n_seqs = frames = padded = 0
    max_b = 0
    for batch in batches:
        lens = [b[args.key].shape[0] for b in batch]
        n_batches += 1
        n_seqs += len(batch)
        frames += sum(lens)
        padded += max(lens) * len(lens)
        max_b = max(max_b, len(batch))
    print("batches: %i, seqs: %i (max %i per batch, mean %.1f)" % (n_batches, n_seqs, max_b, n_seqs / max(n_batches, 1)))
    print("frames: %i, padded frames: %i, padding ratio: %.2f%%" % (frames, padded, 100.0 * (1.0 - frames / max(padded, 1))))


if __name__ == "__main__":
    sys.exit(main())
