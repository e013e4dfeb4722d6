"""
Fused log-mel frontend (``csrc/mel.cu``): framing, Hann window, DFT, power spectrum, mel projection and log in one
kernel, fp32. The window and the filterbank are built once per configuration with the same formulas as the RF path
(:mod:`returnn_b200.frontend.audio.mel`, :func:`returnn_b200.frontend.signal.stft`), so both give the same features.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import math
import torch
from . import _lib

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_cache = {}


def available() -> bool:
    """library present with the entry point"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_log_mel")


def _tables(device, sampling_rate, window, n_fft, n_mel, f_min, f_max):
    key = (str(device), sampling_rate, window, n_fft, n_mel, f_min, f_max)
    t = _cache.get(key)
    if t is None:
        from ..frontend.audio.mel import _fbank_matrix

        win_len = window - (window % 2)
        win = torch.hann_window(win_len, periodic=True, dtype=torch.float32)
        if win_len < window:
            win = torch.nn.functional.pad(win, [0, window - win_len])
        fb = torch.from_numpy(_fbank_matrix(int(sampling_rate), n_fft, f_min, f_max, n_mel))
        t = (win.to(device).contiguous(), fb.to(device).contiguous())
        _cache[key] = t
    return t


def log_mel(audio: torch.Tensor, *, sampling_rate: int, window: int, step: int, n_fft: int, n_mel: int, f_min: float, f_max: float,
            log_base: float = 10.0, lens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """
    :param audio: [..., samples] on a CUDA device (any float dtype; converted to fp32)
    :param lens: [rows] valid samples per row (frames beyond are zero)
    :return: [..., n_frames, n_mel] fp32, ``n_frames = (samples - window) // step + 1``
    """
    shape = list(audio.shape)
    flat = audio.reshape(-1, shape[-1]).float().contiguous()
    rows, T = flat.shape
    n_frames = (T - window) // step + 1 if T >= window else 0
    out = torch.zeros(rows, n_frames, n_mel, dtype=torch.float32, device=audio.device)
    if n_frames > 0:
        win, fb = _tables(audio.device, sampling_rate, window, n_fft, n_mel, f_min, f_max)
        l32 = lens.to(audio.device, torch.int32).contiguous() if lens is not None else None
        fn = _lib.bind("rb200_log_mel", [_vp, _vp, _i32, _i64, _i32, _i32, _i32, _vp, _vp, _i32, _f32, _f32, _vp, _vp])
        scale = 1.0 if log_base == math.e else 1.0 / math.log(log_base)
        _lib.check(fn(flat.data_ptr(), l32.data_ptr() if l32 is not None else None, rows, T, window, step, n_fft, win.data_ptr(), fb.data_ptr(), n_mel,
                      scale, 1e-10, out.data_ptr(), _lib.stream_ptr()), "log_mel")
        _lib.count_launch()
    return out.reshape(shape[:-1] + [n_frames, n_mel])
