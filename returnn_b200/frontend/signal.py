"""
Signal processing: STFT.  Parity: returnn/frontend/signal.py; returnn/torch/frontend/_backend.py:2634-2715
(Hann window, centered frames off by default = "valid" framing like TF, fp32 upcast for bf16).
"""

from __future__ import annotations
from typing import Optional, Tuple
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap, axis_of

__all__ = ["stft"]


def stft(x: Tensor, *, in_spatial_dim: Dim, frame_step: int, frame_length: int, fft_length: Optional[int] = None,
         window_use_frame_length: bool = True, align_window_left: bool = True, window_enforce_even: bool = True,
         out_spatial_dim: Optional[Dim] = None, out_dim: Optional[Dim] = None) -> Tuple[Tensor, Dim, Dim]:
    """
    Short-time Fourier transform. Frames start at ``t * frame_step`` (no centering / no padding: T_out =
    (T - frame_length) // frame_step + 1). Hann window of frame_length, zero-padded to fft_length.

    :return: complex64 [.., out_spatial_dim, out_dim = fft_length//2+1], out_spatial_dim, out_dim
    """
    if fft_length is None:
        fft_length = frame_length
    if out_dim is None:
        out_dim = Dim(fft_length // 2 + 1, name="stft-freq")
    if out_spatial_dim is None:
        out_spatial_dim = Dim._derive("conv", [in_spatial_dim], attribs={"filter_size": frame_length, "stride": frame_step, "dilation": 1, "padding": "valid"})
    rest = [d for d in x._dims if d != in_spatial_dim]
    raw = x.copy_compatible_to_dims_raw(rest + [in_spatial_dim])
    if raw.dtype in (torch.bfloat16, torch.float16):
        raw = raw.float()
    shape = list(raw.shape)
    flat = raw.reshape(-1, shape[-1])
    T = shape[-1]
    n_frames = max((T - frame_length) // frame_step + 1, 0) if T >= frame_length else 0
    win_len = frame_length
    if window_enforce_even and win_len % 2 == 1:
        win_len -= 1
    window = torch.hann_window(win_len, periodic=True, dtype=flat.dtype, device=flat.device)
    if win_len < frame_length:
        window = torch.nn.functional.pad(window, [0, frame_length - win_len])
    if n_frames > 0:
        frames = flat.unfold(-1, frame_length, frame_step) * window  # [N, n_frames, frame_length]
        if fft_length > frame_length:
            if align_window_left:
                frames = torch.nn.functional.pad(frames, [0, fft_length - frame_length])
            else:
                left = (fft_length - frame_length) // 2
                frames = torch.nn.functional.pad(frames, [left, fft_length - frame_length - left])
        spec = torch.fft.rfft(frames, n=fft_length, dim=-1)
    else:
        spec = torch.zeros(flat.shape[0], 0, fft_length // 2 + 1, dtype=torch.complex64, device=flat.device)
    spec = spec.reshape(shape[:-1] + [n_frames, fft_length // 2 + 1])
    return wrap(spec, rest + [out_spatial_dim, out_dim], feature_dim=out_dim), out_spatial_dim, out_dim
