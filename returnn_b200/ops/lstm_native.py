"""
Binding of the LSTM recurrence executor (``csrc/lstm.cu``): one native call runs the whole time loop of one direction
(recurrent projection on the tcgen05 GEMM + fused cell kernel per step), forward or backward. The input projection for all
frames is one GEMM through :mod:`returnn_b200.ops.linear` in front of it, the weight gradient of the recurrent matrix one
split-K GEMM after the backward loop.
"""

from __future__ import annotations
import ctypes
from typing import Optional
import torch
from . import _lib
from . import gemm as _gemm

_vp, _i32 = ctypes.c_void_p, ctypes.c_int


def available(x) -> bool:
    """library present with the LSTM entry points"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_lstm_fwd") and x.is_cuda and _gemm.ENABLED


def supports(x, w_rec) -> bool:
    """shapes handled: hidden size and input size multiples of 8 (TMA pitch), at least one frame"""
    H = w_rec.shape[1]
    return H % 8 == 0 and x.shape[-1] % 8 == 0 and x.shape[0] > 0 and x.dtype in (torch.float32, torch.bfloat16)


class _LstmRecFn(torch.autograd.Function):
    """recurrence on pre-projected inputs z_in [T,B,4H]"""

    @staticmethod
    def forward(ctx, z_in, w_rec, lens, h0, c0, reverse):
        T, B, H4 = z_in.shape
        H = H4 // 4
        dev = z_in.device
        z16 = z_in.to(torch.bfloat16).contiguous()
        w16 = w_rec.to(torch.bfloat16).contiguous()
        bf = torch.bfloat16
        y = torch.empty(T, B, H, dtype=bf, device=dev)
        c_all = torch.empty(T, B, H, dtype=torch.float32, device=dev)
        gates = torch.empty(T, B, H4, dtype=bf, device=dev)
        hprev = torch.empty(T, B, H, dtype=bf, device=dev)
        h_fin = torch.empty(B, H, dtype=torch.float32, device=dev)
        c_fin = torch.empty(B, H, dtype=torch.float32, device=dev)
        z_rec = torch.empty(B, H4, dtype=torch.float32, device=dev)
        h_state = torch.empty(B, H, dtype=bf, device=dev)
        h0f, c0f = h0.float().contiguous(), c0.float().contiguous()
        st = _gemm.status_tensor(dev)
        nl = ctypes.c_int(0)
        fn = _lib.bind("rb200_lstm_fwd", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp])
        _lib.check(fn(z16.data_ptr(), w16.data_ptr(), lens.data_ptr() if lens is not None else None, h0f.data_ptr(), c0f.data_ptr(), T, B, H,
                      1 if reverse else 0, y.data_ptr(), c_all.data_ptr(), gates.data_ptr(), hprev.data_ptr(), h_fin.data_ptr(), c_fin.data_ptr(),
                      z_rec.data_ptr(), h_state.data_ptr(), st.data_ptr(), ctypes.addressof(nl), _lib.stream_ptr()), "lstm_fwd")
        _lib.count_launch(nl.value)
        ctx.save_for_backward(w16, lens, gates, c_all, c0f, hprev)
        ctx.meta = (T, B, H, bool(reverse), z_in.dtype, w_rec.dtype, h0.dtype, c0.dtype)
        ctx.mark_non_differentiable()
        return y.to(z_in.dtype) if z_in.dtype != bf else y, h_fin.to(h0.dtype), c_fin.to(c0.dtype)

    @staticmethod
    def backward(ctx, dy, dh_fin, dc_fin):
        w16, lens, gates, c_all, c0f, hprev = ctx.saved_tensors
        T, B, H, reverse, z_dtype, w_dtype, h_dtype, c_dtype = ctx.meta
        dev = gates.device
        dy16 = dy.to(torch.bfloat16).contiguous() if dy is not None else None
        dz = torch.empty(T, B, 4 * H, dtype=torch.bfloat16, device=dev)
        dw = torch.zeros(4 * H, H, dtype=torch.float32, device=dev)
        dh0 = torch.empty(B, H, dtype=torch.float32, device=dev)
        dc0 = torch.empty(B, H, dtype=torch.float32, device=dev)
        dhf = dh_fin.float().contiguous() if dh_fin is not None else None
        dcf = dc_fin.float().contiguous() if dc_fin is not None else None
        st = _gemm.status_tensor(dev)
        nl = ctypes.c_int(0)
        fn = _lib.bind("rb200_lstm_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp])
        _lib.check(fn(dy16.data_ptr() if dy16 is not None else None, dhf.data_ptr() if dhf is not None else None,
                      dcf.data_ptr() if dcf is not None else None, w16.data_ptr(), lens.data_ptr() if lens is not None else None, gates.data_ptr(),
                      c_all.data_ptr(), c0f.data_ptr(), hprev.data_ptr(), T, B, H, 1 if reverse else 0, dz.data_ptr(), dw.data_ptr(), dh0.data_ptr(),
                      dc0.data_ptr(), st.data_ptr(), ctypes.addressof(nl), _lib.stream_ptr()), "lstm_bwd")
        _lib.count_launch(nl.value)
        return dz.to(z_dtype), dw.to(w_dtype), None, dh0.to(h_dtype), dc0.to(c_dtype), None


def lstm(x, lens: Optional[torch.Tensor], w_ff, w_rec, bias, h0, c0, reverse: bool = False):
    """
    :param x: [T, B, in]; w_ff [4H, in], w_rec [4H, H], bias [4H] or None (gate order i, f, g, o)
    :return: y [T, B, H], h_T [B, H], c_T [B, H]
    """
    from . import linear as _lin

    T, B, _ = x.shape
    z_in = _lin.linear(x.to(torch.bfloat16), w_ff.t().to(torch.bfloat16), bias.to(torch.bfloat16) if bias is not None else None)
    l32 = lens.to(x.device, torch.int32).contiguous() if lens is not None else None
    y, h, c = _LstmRecFn.apply(z_in, w_rec, l32, h0, c0, bool(reverse))
    return y.to(x.dtype), h, c
