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
from ..tensor.utils import host_to_device

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
    l32 = host_to_device(lens.to(torch.int32), x.device).contiguous() if lens is not None else None
    y, h, c = _LstmRecFn.apply(z_in, w_rec, l32, h0, c0, bool(reverse))
    return y.to(x.dtype), h, c


def blstm_supported(x, w_rec_fw, w_rec_bw) -> bool:
    """both directions of one layer can run in ONE cooperative launch (two CTAs per SM): same sizes, persistent-kernel shapes"""
    lib = _lib.get_lib()
    if lib is None or not hasattr(lib, "rb200_blstm_fwd") or not available(x):
        return False
    if w_rec_fw.shape != w_rec_bw.shape or not supports(x, w_rec_fw):
        return False
    T, B, _ = x.shape
    fn = _lib.bind("rb200_blstm_supported", [_i32, _i32, _i32])
    return bool(fn(int(T), int(B), int(w_rec_fw.shape[1])))


def persist_supported(x, batch: int, w_rec) -> bool:
    """whether a batch of ``batch`` sequences of this input runs in the persistent recurrence kernels"""
    lib = _lib.get_lib()
    if lib is None or not hasattr(lib, "rb200_blstm_supported") or not available(x) or not supports(x, w_rec):
        return False
    fn = _lib.bind("rb200_blstm_supported", [_i32, _i32, _i32])
    return bool(fn(int(x.shape[0]), int(batch), int(w_rec.shape[1])))


class _BlstmRecFn(torch.autograd.Function):
    """the recurrences of both directions on pre-projected inputs z [T,B,4H], one kernel for the two time loops"""

    @staticmethod
    def forward(ctx, z_fw, z_bw, w_fw, w_bw, lens, h0_fw, c0_fw, h0_bw, c0_bw):
        T, B, H4 = z_fw.shape
        H = H4 // 4
        dev = z_fw.device
        bf = torch.bfloat16
        per_dir = []
        ptrs = (ctypes.c_void_p * 22)()
        keep = []
        for d, (z, w, h0, c0) in enumerate(((z_fw, w_fw, h0_fw, c0_fw), (z_bw, w_bw, h0_bw, c0_bw))):
            z16 = z.to(bf).contiguous()
            w16 = w.to(bf).contiguous()
            y = torch.empty(T, B, H, dtype=bf, device=dev)
            c_all = torch.empty(T, B, H, dtype=torch.float32, device=dev)
            gates = torch.empty(T, B, H4, dtype=bf, device=dev)
            hprev = torch.empty(T, B, H, dtype=bf, device=dev)
            h_fin = torch.empty(B, H, dtype=torch.float32, device=dev)
            c_fin = torch.empty(B, H, dtype=torch.float32, device=dev)
            hbuf = torch.empty(2, B, H, dtype=bf, device=dev)
            h0f, c0f = h0.float().contiguous(), c0.float().contiguous()
            for i, t in enumerate((z16, w16, h0f, c0f, y, c_all, gates, hprev, h_fin, c_fin, hbuf)):
                ptrs[d * 11 + i] = t.data_ptr()
            keep.append((z16, hbuf))
            per_dir.append((w16, gates, c_all, c0f, hprev, y, h_fin, c_fin))
        st = _gemm.status_tensor(dev)
        fn = _lib.bind("rb200_blstm_fwd", [_vp, _vp, _i32, _i32, _i32, _vp, _vp])
        _lib.check(fn(ctypes.cast(ptrs, _vp), lens.data_ptr() if lens is not None else None, T, B, H, st.data_ptr(), _lib.stream_ptr()), "blstm_fwd")
        _lib.count_launch(3)
        (w16f, gf, caf, c0ff, hpf, yf, hff, cff), (w16b, gb, cab, c0fb, hpb, yb, hfb, cfb) = per_dir
        ctx.save_for_backward(lens, w16f, gf, caf, c0ff, hpf, w16b, gb, cab, c0fb, hpb)
        ctx.meta = (T, B, H, z_fw.dtype, w_fw.dtype, h0_fw.dtype, c0_fw.dtype)
        zd = z_fw.dtype
        return (yf.to(zd) if zd != bf else yf, yb.to(zd) if zd != bf else yb, hff.to(h0_fw.dtype), cff.to(c0_fw.dtype),
                hfb.to(h0_bw.dtype), cfb.to(c0_bw.dtype))

    @staticmethod
    def backward(ctx, dy_fw, dy_bw, dh_fw, dc_fw, dh_bw, dc_bw):
        lens, *rest = ctx.saved_tensors
        T, B, H, z_dtype, w_dtype, h_dtype, c_dtype = ctx.meta
        dev = rest[1].device
        bf = torch.bfloat16
        ptrs = (ctypes.c_void_p * 24)()
        outs, keep = [], []
        for d, (dy, dhf, dcf) in enumerate(((dy_fw, dh_fw, dc_fw), (dy_bw, dh_bw, dc_bw))):
            w16, gates, c_all, c0f, hprev = rest[d * 5: d * 5 + 5]
            dy16 = dy.to(bf).contiguous() if dy is not None else None
            dhf32 = dhf.float().contiguous() if dhf is not None else None
            dcf32 = dcf.float().contiguous() if dcf is not None else None
            dz = torch.empty(T, B, 4 * H, dtype=bf, device=dev)
            dw = torch.zeros(4 * H, H, dtype=torch.float32, device=dev)
            dh0 = torch.empty(B, H, dtype=torch.float32, device=dev)
            dc0 = torch.empty(B, H, dtype=torch.float32, device=dev)
            for i, t in enumerate((dy16, dhf32, dcf32, w16, gates, c_all, c0f, hprev, dz, dw, dh0, dc0)):
                ptrs[d * 12 + i] = t.data_ptr() if t is not None else None
            keep.append((dy16, dhf32, dcf32))
            outs.append((dz, dw, dh0, dc0))
        st = _gemm.status_tensor(dev)
        nl = ctypes.c_int(0)
        fn = _lib.bind("rb200_blstm_bwd", [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp])
        _lib.check(fn(ctypes.cast(ptrs, _vp), lens.data_ptr() if lens is not None else None, T, B, H, st.data_ptr(), ctypes.addressof(nl),
                      _lib.stream_ptr()), "blstm_bwd")
        _lib.count_launch(nl.value)
        (dzf, dwf, dh0f, dc0f), (dzb, dwb, dh0b, dc0b) = outs
        return (dzf.to(z_dtype), dzb.to(z_dtype), dwf.to(w_dtype), dwb.to(w_dtype), None, dh0f.to(h_dtype), dc0f.to(c_dtype),
                dh0b.to(h_dtype), dc0b.to(c_dtype))


def blstm(x, lens: Optional[torch.Tensor], fw, bw, h0_fw, c0_fw, h0_bw, c0_bw):
    """
    Forward-in-time and reversed LSTM over the same input, both recurrences in one kernel.

    :param x: [T, B, in]
    :param fw: (w_ff [4H, in], w_rec [4H, H], bias [4H] or None) of the forward direction; ``bw`` likewise for the reversed one
    :return: (y_fw [T,B,H], h_T, c_T), (y_bw [T,B,H], h_T, c_T)
    """
    from . import linear as _lin

    bf = torch.bfloat16
    x16 = x.to(bf)
    zs = []
    for w_ff, _w_rec, bias in (fw, bw):
        zs.append(_lin.linear(x16, w_ff.t().to(bf), bias.to(bf) if bias is not None else None))
    l32 = host_to_device(lens.to(torch.int32), x.device).contiguous() if lens is not None else None
    yf, yb, hf, cf, hb, cb = _BlstmRecFn.apply(zs[0], zs[1], fw[1], bw[1], l32, h0_fw, c0_fw, h0_bw, c0_bw)
    return (yf.to(x.dtype), hf, cf), (yb.to(x.dtype), hb, cb)
