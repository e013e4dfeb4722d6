"""Decoder zoo: Transformer decoder."""

from . import transformer
