"""
Conformer v2: same blocks, with the ESPnet-style defaults (input embedding scale sqrt(D), final layer norm optional).
Parity: returnn/frontend/encoder/conformer_v2.py.
"""

from __future__ import annotations
from typing import Optional
from ...tensor import Tensor, Dim
from .conformer import ConformerEncoder, ConformerEncoderLayer, ConformerConvSubsample, ConformerConvBlock

__all__ = ["ConformerEncoderV2", "ConformerEncoderLayerV2"]


class ConformerEncoderLayerV2(ConformerEncoderLayer):
    """v2 block: identical computation; kept as a separate class for config compatibility"""


class ConformerEncoderV2(ConformerEncoder):
    """v2 encoder: default ``input_embedding_scale = sqrt(out_dim)`` regardless of pos_enc"""

    def __init__(self, in_dim: Dim, out_dim=Dim(512, name="conformer-enc-default-out-dim"), *, input_embedding_scale: Optional[float] = None, **kwargs):
        if input_embedding_scale is None:
            d = out_dim if isinstance(out_dim, int) else out_dim.dimension
            input_embedding_scale = d ** 0.5
        kwargs.setdefault("encoder_layer", ConformerEncoderLayerV2)
        super().__init__(in_dim, out_dim, input_embedding_scale=input_embedding_scale, **kwargs)
