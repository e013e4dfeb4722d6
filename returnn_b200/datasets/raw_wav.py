"""
:class:`RawWavDataset`: the raw waveform of wav files as input sequences, cut into frames of ``frameLength`` samples every
``frameShift`` samples (the last frame zero-padded). ``listFile`` names one wav file per line; a line may name a second file after
whitespace, whose frames become the regression target ``classes``. Decoded signals are kept in memory after first use.
Reference: returnn/datasets/raw_wav.py (which buffers in a temporary HDF file instead).
"""

from __future__ import annotations
from typing import Dict, List, Optional, Tuple
import numpy
from .basic import DatasetSeq
from .cached2 import CachedDataset2


class RawWavDataset(CachedDataset2):
    """frames of raw samples"""

    def __init__(self, listFile: str, frameLength: int, frameShift: int, num_outputs: Optional[int] = None, **kwargs):
        super().__init__(**kwargs)
        with open(listFile) as f:
            self._wavFiles: List[Tuple[str, Optional[str]]] = []
            for line in f:
                parts = line.split()
                if parts:
                    self._wavFiles.append((parts[0], parts[1] if len(parts) > 1 else None))
        self._frameLength, self._frameShift = int(frameLength), int(frameShift)
        self._flag_pad = True
        self._buffer: Dict[str, numpy.ndarray] = {}
        self._seq_index_list: List[int] = []
        self.num_inputs = self._frameLength
        has_targets = any(t is not None for _, t in self._wavFiles)
        if not has_targets and num_outputs is None:
            raise ValueError("If no output data is used, num_outputs needs to be set for RawWavDataset")
        self.num_outputs = {"data": (self._frameLength, 2), "classes": (self._frameLength if has_targets else int(num_outputs), 2)}
        self._has_targets = has_targets

    def _signal(self, path: str) -> numpy.ndarray:
        if path not in self._buffer:
            from .audio import read_audio

            with open(path, "rb") as f:
                audio, _sr = read_audio(f.read(), path if path.lower().endswith(".wav") else path + ".wav")
            self._buffer[path] = audio if audio.ndim == 1 else audio.mean(axis=1)
        return self._buffer[path]

    def _frames(self, signal: numpy.ndarray) -> numpy.ndarray:
        n, length, shift = signal.shape[0], self._frameLength, self._frameShift
        num = max(int(numpy.ceil(float(n - length) / shift + 1)), 1)
        if self._flag_pad:
            padded = numpy.zeros(((num - 1) * shift + length,), dtype="float32")
            padded[:n] = signal[: padded.shape[0]]
        else:
            num = max(num - 1, 1)
            padded = signal[: (num - 1) * shift + length]
        idx = numpy.arange(num)[:, None] * shift + numpy.arange(length)[None, :]
        return padded[idx].astype("float32")

    def get_total_num_seqs(self, *, fast: bool = False) -> int:
        return len(self._wavFiles)

    def init_seq_order(self, epoch=None, seq_list=None, seq_order=None):
        super().init_seq_order(epoch=epoch, seq_list=seq_list, seq_order=seq_order)
        if seq_order is not None:
            self._seq_index_list = list(seq_order)
        else:
            self._seq_index_list = list(self.get_seq_order_for_epoch(epoch or 1, len(self._wavFiles), lambda i: self._signal(self._wavFiles[i][0]).shape[0]))
        self._num_seqs = len(self._seq_index_list)
        return True

    @property
    def num_seqs(self) -> int:
        return len(self._seq_index_list)

    def _collect_single_seq(self, seq_idx: int) -> Optional[DatasetSeq]:
        if seq_idx >= len(self._seq_index_list):
            return None
        wav_id = self._seq_index_list[seq_idx]
        src, tgt = self._wavFiles[wav_id]
        x = self._frames(self._signal(src))
        y = self._frames(self._signal(tgt)) if tgt is not None else None
        return DatasetSeq(seq_idx=seq_idx, seq_tag="wav-%i" % wav_id, features=x, targets=y)

    def get_data_keys(self):
        return ["data", "classes"] if self._has_targets else ["data"]

    def get_target_list(self):
        return ["classes"] if self._has_targets else []

    def get_data_dtype(self, key):
        return "float32"

    def is_data_sparse(self, key):
        return False
