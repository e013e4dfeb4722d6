#!/usr/bin/env python3
"""Iterate over a dataset given as a dict on the command line and print shapes, e.g. '{"class": "Task12AXDataset", "num_seqs": 3}'"""

import sys
import _setup_env  # noqa: F401
from returnn_b200.datasets.basic import init_dataset


def main():
    opts = eval(sys.argv[1]) if len(sys.argv) > 1 else {"class": "Task12AXDataset", "num_seqs": 3}
    ds = init_dataset(opts)
    ds.init_seq_order(epoch=1)
    seq_idx = 0
    while ds.is_less_than_num_seqs(seq_idx):
        ds.load_seqs(seq_idx, seq_idx + 1)
        print(seq_idx, ds.get_tag(seq_idx), {k: ds.get_data(seq_idx, k).shape for k in ds.get_data_keys()})
        seq_idx += 1


if __name__ == "__main__":
    main()
