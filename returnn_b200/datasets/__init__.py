"""
Datasets. ``init_dataset({"class": "<Name>", ...})`` looks the class up over all modules in this package.
"""

from .basic import Dataset, DatasetSeq, init_dataset, init_dataset_via_str, get_dataset_class
