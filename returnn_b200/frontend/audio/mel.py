"""
Mel filterbank features.

Parity: returnn/frontend/audio/mel.py:18-208 (mel_filterbank :18-76, log_mel_filterbank_from_raw :163-208:
n_fft = next power of two of the window, power spectrum, mel matmul, log10 with floor).
"""

from __future__ import annotations
from typing import Optional, Tuple, Union
import math
import numpy
import torch
from ...tensor import Tensor, Dim
from .._utils import wrap
from ..signal import stft
from ..matmul import matmul
from .. import math_ as _m

__all__ = ["mel_filterbank", "log_mel_filterbank_from_raw"]

_fbank_cache = {}


def _hz_to_mel(f):
    return 1127.0 * numpy.log1p(numpy.asarray(f, dtype="float64") / 700.0)


def _mel_to_hz(m):
    return 700.0 * (numpy.exp(numpy.asarray(m, dtype="float64") / 1127.0) - 1.0)


def _fbank_matrix(sampling_rate: int, fft_length: int, f_min: float, f_max: float, nr_of_filters: int) -> numpy.ndarray:
    """triangular filters equally spaced on the mel scale (HTK formula): [fft_length//2+1, nr_of_filters]"""
    n_bins = fft_length // 2 + 1
    mel_pts = numpy.linspace(_hz_to_mel(f_min), _hz_to_mel(f_max), nr_of_filters + 2)
    bin_mel = _hz_to_mel(numpy.linspace(0.0, sampling_rate / 2.0, n_bins))
    fb = numpy.zeros((n_bins, nr_of_filters), dtype="float32")
    for i in range(nr_of_filters):
        lo, ce, hi = mel_pts[i], mel_pts[i + 1], mel_pts[i + 2]
        up = (bin_mel - lo) / (ce - lo)
        down = (hi - bin_mel) / (hi - ce)
        fb[:, i] = numpy.maximum(0.0, numpy.minimum(up, down))
    return fb


def mel_filterbank(x: Tensor, *, in_dim: Dim, out_dim: Dim, sampling_rate: Union[int, float], fft_length: Optional[int] = None,
                   f_min: Optional[float] = None, f_max: Optional[float] = None) -> Tensor:
    """apply the mel filterbank to a (power) spectrum over in_dim"""
    if fft_length is None:
        fft_length = (in_dim.dimension - 1) * 2
    f_min = f_min or 0
    f_max = f_max or sampling_rate / 2.0
    key = (sampling_rate, fft_length, f_min, f_max, out_dim.dimension, x.dtype, x.device)
    fb = _fbank_cache.get(key)
    if fb is None:
        mat = _fbank_matrix(int(sampling_rate), fft_length, f_min, f_max, out_dim.dimension)
        fb = torch.from_numpy(mat).to(x.raw_tensor.dtype).to(x.raw_tensor.device)
        _fbank_cache[key] = fb
    return matmul(x, wrap(fb, [in_dim, out_dim]), reduce=in_dim)


def log_mel_filterbank_from_raw(raw_audio: Tensor, *, in_spatial_dim: Dim, out_dim: Dim, sampling_rate: int = 16000,
                                window_len: float = 0.025, step_len: float = 0.010, n_fft: Optional[int] = None,
                                log_base: Union[int, float] = 10, f_min=None, f_max=None, mel_normalization: bool = False) -> Tuple[Tensor, Dim]:
    """
    :param raw_audio: [.., in_spatial_dim] samples
    :return: [.., out_spatial_dim, out_dim] log-mel features, out_spatial_dim
    """
    if raw_audio.feature_dim and raw_audio.feature_dim.dimension == 1:
        from ..array_ import squeeze

        raw_audio = squeeze(raw_audio, axis=raw_audio.feature_dim)
    window_num_frames = int(window_len * sampling_rate)
    step_num_frames = int(step_len * sampling_rate)
    if not n_fft:
        n_fft = 1 << (window_num_frames - 1).bit_length()
    if raw_audio.raw_tensor.is_cuda:
        from ...ops import logmel as _lm

        if _lm.available():
            rest = [d for d in raw_audio.dims if d != in_spatial_dim]
            from ..conv import make_conv_out_spatial_dims

            (osd,) = make_conv_out_spatial_dims([in_spatial_dim], filter_size=window_num_frames, strides=step_num_frames, padding="valid")
            out = _lm.log_mel(raw_audio.copy_compatible_to_dims_raw(rest + [in_spatial_dim]), sampling_rate=sampling_rate,
                              window=window_num_frames, step=step_num_frames, n_fft=n_fft, n_mel=out_dim.dimension,
                              f_min=f_min or 0.0, f_max=f_max or sampling_rate / 2.0, log_base=log_base)
            return wrap(out, rest + [osd, out_dim], feature_dim=out_dim), osd
    spectrogram, out_spatial_dim, in_dim_ = stft(raw_audio, in_spatial_dim=in_spatial_dim, frame_step=step_num_frames,
                                                 frame_length=window_num_frames, fft_length=n_fft)
    power = wrap(spectrogram.raw_tensor.abs().square(), spectrogram.dims, feature_dim=in_dim_)
    mel = mel_filterbank(power, in_dim=in_dim_, out_dim=out_dim, sampling_rate=sampling_rate, fft_length=n_fft, f_min=f_min, f_max=f_max)
    log_mel = _m.safe_log(mel, eps=1e-10)
    if log_base != math.e:
        log_mel = log_mel * (1.0 / math.log(log_base))
    return log_mel, out_spatial_dim
