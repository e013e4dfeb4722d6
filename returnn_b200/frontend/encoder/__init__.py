"""Encoder zoo: Conformer (v1/v2), E-Branchformer, Transformer encoder."""

from . import base, conformer, conformer_v2, e_branchformer, transformer
