"""
Bundle file: a text file that lists, one path per line, the HDF files that together form a corpus (used by the stereo datasets
when ``hdfFile`` ends in ``.bundle``).  Reference: returnn/datasets/bundle_file.py.
"""

from __future__ import annotations
from typing import List


class BundleFile:
    """the paths listed in a bundle file"""

    def __init__(self, file_path: str):
        self._file_path = file_path
        with open(file_path, "r") as f:
            self._paths: List[str] = [line.strip() for line in f if line.strip()]

    @property
    def dataset_file_paths(self) -> List[str]:
        """paths of the dataset files, in file order"""
        return list(self._paths)

    @property
    def number_of_dataset_files(self) -> int:
        """how many"""
        return len(self._paths)
