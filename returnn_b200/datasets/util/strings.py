"""String helpers of the dataset layer. Parity: returnn/datasets/util/strings.py."""

from __future__ import annotations
import numpy


def str_to_numpy_array(s: str) -> numpy.ndarray:
    """the canonical array form of a Python string in a ``Tensor``: a 0-d array of kind ``U``"""
    return numpy.array(s)
