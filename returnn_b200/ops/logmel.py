"""
Log-mel frontend on own kernels (``csrc/mel.cu``): framing, Hann window, DFT, power spectrum, mel projection, log.
The window and the filterbank are built once per configuration with the same formulas as the RF path
(:mod:`returnn_b200.frontend.audio.mel`, :func:`returnn_b200.frontend.signal.stft`), so both give the same features.

Two forms. Large inputs run the DFT on the tensor cores: all frames times the windowed cos / sin table is one matrix product on the
tcgen05 GEMM, with the frames read as an overlapping strided view of the audio (no frame matrix in memory), fp32 precision kept by
splitting both factors into fp16 high and low parts (three accumulating products, 22 mantissa bits per factor), followed by one kernel for power -> mel -> log.
Small inputs (or a hop size that is not a multiple of 8 samples, which the strided view needs for 16-byte row pitches) run the
single fp32 kernel that does everything per block of 8 frames.
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


def _dft_tables(device, window: int, n_fft: int, win: torch.Tensor, fb: torch.Tensor):
    """
    (table_hi, table_lo) fp16 [window, n_fft]: column 2j = win * cos(2 pi j n / n_fft), 2j + 1 = -win * sin(..) for 0 < j < n_fft/2,
    column 0 = win (X_0) and column 1 = win * (-1)^n (X_{n_fft/2}); and the non-zero bin range of every mel filter.
    """
    key = ("dft", str(device), window, n_fft, win.data_ptr(), fb.data_ptr())
    t = _cache.get(key)
    if t is None:
        n = torch.arange(window, dtype=torch.float64)[:, None]
        j = torch.arange(n_fft // 2, dtype=torch.float64)[None, :]
        ang = 2.0 * math.pi * ((n * j) % n_fft) / n_fft
        w64 = win.double().cpu()[:, None]
        table = torch.empty(window, n_fft, dtype=torch.float64)
        table[:, 0::2] = torch.cos(ang) * w64
        table[:, 1::2] = -torch.sin(ang) * w64
        table[:, 1] = (w64 * torch.cos(math.pi * n))[:, 0]
        table = table.float()
        hi = table.half()
        lo = (table - hi.float()).half()
        nz = fb.cpu() != 0  # [n_bins, n_mel]
        idx = torch.arange(nz.shape[0])[:, None].expand_as(nz)
        big = nz.shape[0]
        start = torch.where(nz, idx, torch.full_like(idx, big)).min(dim=0).values
        end = torch.where(nz, idx + 1, torch.zeros_like(idx)).max(dim=0).values
        length = torch.clamp(end - start, min=0)
        start = torch.where(length > 0, start, torch.zeros_like(start))
        t = (hi.to(device).contiguous(), lo.to(device).contiguous(), start.to(device, torch.int32).contiguous(), length.to(device, torch.int32).contiguous())
        _cache[key] = t
    return t


def _gemm_form_wanted(flat: torch.Tensor, window: int, step: int, n_fft: int) -> bool:
    import os
    from . import gemm as G

    mode = os.environ.get("RETURNN_B200_LOGMEL", "auto")
    if mode == "direct" or step % 8 != 0 or n_fft % 16 != 0 or window > n_fft or n_fft > 8192:
        return False
    lib = _lib.get_lib()
    if lib is None or not hasattr(lib, "rb200_mel_from_spectrum") or not G.available(flat):
        return False
    rows, T = flat.shape
    return mode == "gemm" or rows * (T // step) >= 2048


def _log_mel_gemm(flat: torch.Tensor, l32, *, window, step, n_fft, n_mel, win, fb, scale, n_frames, out):
    from . import gemm as G

    rows, T = flat.shape
    dev = flat.device
    slots = -(-T // step)
    Tp = slots * step
    total = rows * Tp + ((window + 7) // 8) * 8  # the last slots read up to `window` samples past the last row
    hi = torch.empty(total, dtype=torch.float16, device=dev)
    lo = torch.empty(total, dtype=torch.float16, device=dev)
    fn = _lib.bind("rb200_split_hi_lo_fp16", [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp])
    _lib.check(fn(flat.data_ptr(), rows, T, Tp, total, hi.data_ptr(), lo.data_ptr(), _lib.stream_ptr()), "split_hi_lo")
    t_hi, t_lo, fb_start, fb_len = _dft_tables(dev, window, n_fft, win, fb)
    m = rows * slots
    a_hi = torch.as_strided(hi, (m, window), (step, 1))
    a_lo = torch.as_strided(lo, (m, window), (step, 1))
    spec = torch.empty(m, n_fft, dtype=torch.float32, device=dev)
    G.gemm(a_hi, t_hi, m=m, n=n_fft, k=window, a_mn_major=False, b_mn_major=True, out=spec)
    G.gemm(a_hi, t_lo, m=m, n=n_fft, k=window, a_mn_major=False, b_mn_major=True, out=spec, accumulate=True)
    G.gemm(a_lo, t_hi, m=m, n=n_fft, k=window, a_mn_major=False, b_mn_major=True, out=spec, accumulate=True)
    fn = _lib.bind("rb200_mel_from_spectrum", [_vp, _i32, _i32, _i32, _i32, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _f32, _f32, _vp, _vp])
    _lib.check(fn(spec.data_ptr(), n_fft, rows, slots, n_frames, l32.data_ptr() if l32 is not None else None, T, window, step, n_fft, fb.data_ptr(),
                  fb_start.data_ptr(), fb_len.data_ptr(), n_mel, scale, 1e-10, out.data_ptr(), _lib.stream_ptr()), "mel_from_spectrum")
    _lib.count_launch(2)


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
    out = torch.empty(rows, n_frames, n_mel, dtype=torch.float32, device=audio.device)
    if n_frames > 0:
        win, fb = _tables(audio.device, sampling_rate, window, n_fft, n_mel, f_min, f_max)
        l32 = lens.to(audio.device, torch.int32).contiguous() if lens is not None else None
        scale = 1.0 if log_base == math.e else 1.0 / math.log(log_base)
        if _gemm_form_wanted(flat, window, step, n_fft):
            _log_mel_gemm(flat, l32, window=window, step=step, n_fft=n_fft, n_mel=n_mel, win=win, fb=fb, scale=scale, n_frames=n_frames, out=out)
            return out.reshape(shape[:-1] + [n_frames, n_mel])
        fn = _lib.bind("rb200_log_mel", [_vp, _vp, _i32, _i64, _i32, _i32, _i32, _vp, _vp, _i32, _f32, _f32, _vp, _vp])
        _lib.check(fn(flat.data_ptr(), l32.data_ptr() if l32 is not None else None, rows, T, window, step, n_fft, win.data_ptr(), fb.data_ptr(), n_mel,
                      scale, 1e-10, out.data_ptr(), _lib.stream_ptr()), "log_mel")
        _lib.count_launch()
    return out.reshape(shape[:-1] + [n_frames, n_mel])
