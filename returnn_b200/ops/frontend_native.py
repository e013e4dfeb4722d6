"""
Conv2d subsampling frontend on B200 (``csrc/frontend.cu`` + the tcgen05 GEMM): 3x3 convolutions over (time, feature) as
implicit GEMMs with fused bias / ReLU / ReLU-gradient epilogues, the first layer (one input channel) with fused ReLU +
max-pool, the last layer computed directly for the valid frames only (packed rows). One autograd function covers the whole
stack; its backward runs transposed gathers + GEMMs for the data gradients and split-K GEMMs for the filter gradients.

Handles the layout of :class:`returnn_b200.frontend.encoder.conformer.ConformerConvSubsample` with three 3x3 layers,
feature stride 1, "same" padding, pool ``(1, 2)`` after the first layer and ReLU; everything else uses the torch path.
"""

from __future__ import annotations
from typing import List, Optional, Tuple
import ctypes
import torch
from . import _lib
from . import gemm as _gemm

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


def available(x: torch.Tensor) -> bool:
    """library with the frontend entry points, CUDA input"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_im2col_3x3") and x.is_cuda and _gemm.ENABLED


def supports(in_feat: int, channels: Tuple[int, ...], filter_sizes, strides, pool_sizes) -> bool:
    """the geometry the kernels implement"""
    if len(channels) != 3 or any(c % 8 or c > 256 for c in channels) or in_feat % 2 or in_feat % 8:
        return False
    if any(tuple(fs) != (3, 3) for fs in filter_sizes):
        return False
    if tuple(strides[0]) != (1, 1) or any(st[1] != 1 for st in strides):
        return False
    if not pool_sizes or len(pool_sizes) != 1 or tuple(pool_sizes[0]) != (1, 2):
        return False
    return 256 % (channels[0] // 8) == 0


def _same_pad_left(in_len: int, k: int, stride: int) -> int:
    """left part of "same" padding, by the rule rf.conv follows at the current behavior version (from 24 on it no longer depends on
    the padded length of the batch when the convolution has a stride)"""
    from ..frontend.conv import _use_consistent_same_padding

    if stride != 1 and _use_consistent_same_padding():
        return (k - 1) // 2
    pad = max(k - 1 - (in_len - 1) % stride, 0)
    return pad // 2


def _call(name, argtypes, *args):
    fn = _lib.bind(name, argtypes)
    _lib.check(fn(*args), name)
    _lib.count_launch()


def _im2col(x, lens_in, T, F, C, stride, pad, To, row_batch, row_pos, n_frames):
    col = torch.empty(n_frames * F, 9 * C, dtype=torch.bfloat16, device=x.device)
    _call("rb200_im2col_3x3", [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _vp, _vp], x.data_ptr(), lens_in.data_ptr(), T, F, C,
          stride, pad, To, row_batch.data_ptr() if row_batch is not None else None, row_pos.data_ptr() if row_pos is not None else None, n_frames,
          col.data_ptr(), _lib.stream_ptr())
    return col


def _im2col_t(dy, lens_out, lens_in, cu, B, T, F, Co, stride, pad, To):
    col = torch.empty(B * T * F, 9 * Co, dtype=torch.bfloat16, device=dy.device)
    _call("rb200_im2col_3x3_transposed", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp], dy.data_ptr(), lens_out.data_ptr(),
          lens_in.data_ptr(), cu.data_ptr() if cu is not None else None, B, T, F, Co, stride, pad, To, col.data_ptr(), _lib.stream_ptr())
    return col


def _col2im(dcol, lens_out, lens_in, cu, B, T, F, Ci, stride, pad, To, relu_z):
    dx = torch.empty(B, T, F, Ci, dtype=torch.bfloat16, device=dcol.device)
    _call("rb200_col2im_3x3", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp], dcol.data_ptr(), lens_out.data_ptr(),
          lens_in.data_ptr(), cu.data_ptr() if cu is not None else None, B, T, F, Ci, stride, pad, To,
          relu_z.data_ptr() if relu_z is not None else None, dx.data_ptr(), _lib.stream_ptr())
    return dx


def _colsum(x: torch.Tensor) -> torch.Tensor:
    """column sums of a bf16 [rows, C] matrix in fp32 (bias gradient), one pass on the native kernel"""
    lib = _lib.get_lib()
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and lib is not None and hasattr(lib, "rb200_colsum_bf16") and x.shape[1] % 8 == 0:
        out = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        _call("rb200_colsum_bf16", [_vp, _vp, _i32, _i32, _vp], x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _lib.stream_ptr())
        return out
    return x.float().sum(0)


class _FrontendFn(torch.autograd.Function):
    """feats [B,T,F] bf16 -> packed rows [n, (F/2)*C3] bf16"""

    @staticmethod
    def forward(ctx, feats, lens_dev, row_batch, row_pos, cu, w1, b1, w2, b2, w3, b3, s2, s3):
        # lens_dev: int32 [3, B] lengths after conv1 (= input), conv2, conv3
        B, T, F = feats.shape
        C1, C2, C3 = w1.shape[0], w2.shape[0], w3.shape[0]
        Fp = F // 2
        dev = feats.device
        x = feats.contiguous()
        bf = torch.bfloat16
        w1f = w1.float().reshape(C1, 9).contiguous()
        b1f = b1.float().contiguous() if b1 is not None else None
        out1 = torch.empty(B, T, Fp, C1, dtype=bf, device=dev)
        _call("rb200_conv1_relu_pool_fwd", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp], x.data_ptr(), w1f.data_ptr(),
              b1f.data_ptr() if b1f is not None else None, lens_dev[0].data_ptr(), B, T, F, C1, out1.data_ptr(), _lib.stream_ptr())
        # conv2 on the padded batch
        T2 = -(-T // s2)
        pad2 = _same_pad_left(T, 3, s2)
        col2 = _im2col(out1, lens_dev[0], T, Fp, C1, s2, pad2, T2, None, None, B * T2)
        w2p = w2.permute(0, 2, 3, 1).reshape(C2, 9 * C1).to(bf).contiguous()
        out2 = _gemm.gemm(col2, w2p, m=col2.shape[0], n=C2, k=9 * C1, a_mn_major=False, b_mn_major=False, bias=b2.float() if b2 is not None else None,
                          act="relu").view(B, T2, Fp, C2)
        # conv3 for the valid output frames only: the result is already in packed-row order
        T3 = -(-T2 // s3)
        pad3 = _same_pad_left(T2, 3, s3)
        n = row_batch.shape[0]
        col3 = _im2col(out2, lens_dev[1], T2, Fp, C2, s3, pad3, T3, row_batch, row_pos, n)
        w3p = w3.permute(0, 2, 3, 1).reshape(C3, 9 * C2).to(bf).contiguous()
        out3 = _gemm.gemm(col3, w3p, m=col3.shape[0], n=C3, k=9 * C2, a_mn_major=False, b_mn_major=False, bias=b3.float() if b3 is not None else None,
                          act="relu")
        ctx.save_for_backward(x, lens_dev, cu, w1f, b1f, w2, w3, out1, col2, out2, col3, out3)
        ctx.geom = (B, T, F, C1, C2, C3, T2, T3, s2, s3, pad2, pad3, n, b1 is not None, b2 is not None, b3 is not None, w1.dtype)
        return out3.view(n, Fp * C3)

    @staticmethod
    def backward(ctx, d_out):
        x, lens_dev, cu, w1f, b1f, w2, w3, out1, col2, out2, col3, out3 = ctx.saved_tensors
        B, T, F, C1, C2, C3, T2, T3, s2, s3, pad2, pad3, n, has_b1, has_b2, has_b3, wdtype = ctx.geom
        Fp = F // 2
        dev = d_out.device
        bf = torch.bfloat16
        # ---- layer 3
        dz3 = torch.where(out3 > 0, d_out.reshape(n * Fp, C3).to(bf), torch.zeros((), dtype=bf, device=dev)).contiguous()
        dw3p = torch.zeros(C3, 9 * C2, dtype=torch.float32, device=dev)
        _gemm.gemm(dz3, col3, m=C3, n=9 * C2, k=dz3.shape[0], a_mn_major=True, b_mn_major=True, out=dw3p, atomic=True)
        db3 = _colsum(dz3) if has_b3 else None
        # data gradient of layer 3: patch gradients on the output side, gathered back (times relu'(out2))
        w3p = w3.permute(0, 2, 3, 1).reshape(C3, 9 * C2).to(bf).contiguous()
        dcol3 = _gemm.gemm(dz3, w3p, m=dz3.shape[0], n=9 * C2, k=C3, a_mn_major=False, b_mn_major=True)
        dz2 = _col2im(dcol3, lens_dev[2], lens_dev[1], cu, B, T2, Fp, C2, s3, pad3, T3, out2).view(-1, C2)
        del dcol3
        # ---- layer 2
        dw2p = torch.zeros(C2, 9 * C1, dtype=torch.float32, device=dev)
        _gemm.gemm(dz2, col2, m=C2, n=9 * C1, k=dz2.shape[0], a_mn_major=True, b_mn_major=True, out=dw2p, atomic=True)
        db2 = _colsum(dz2) if has_b2 else None
        w2p = w2.permute(0, 2, 3, 1).reshape(C2, 9 * C1).to(bf).contiguous()
        dcol2 = _gemm.gemm(dz2, w2p, m=dz2.shape[0], n=9 * C1, k=C2, a_mn_major=False, b_mn_major=True)
        d_out1 = _col2im(dcol2, lens_dev[1], lens_dev[0], None, B, T, Fp, C1, s2, pad2, T2, None)
        del dcol2
        # ---- layer 1: filter / bias gradient by direct reduction (pool routing and ReLU recomputed)
        dw1 = torch.zeros(C1, 9, dtype=torch.float32, device=dev)
        db1 = torch.zeros(C1, dtype=torch.float32, device=dev) if has_b1 else None
        _call("rb200_conv1_relu_pool_bwd", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp], x.data_ptr(), w1f.data_ptr(),
              b1f.data_ptr() if b1f is not None else None, lens_dev[0].data_ptr(), d_out1.data_ptr(), B, T, F, C1, dw1.data_ptr(),
              db1.data_ptr() if db1 is not None else None, _lib.stream_ptr())
        gw3 = dw3p.view(C3, 3, 3, C2).permute(0, 3, 1, 2).to(wdtype)
        gw2 = dw2p.view(C2, 3, 3, C1).permute(0, 3, 1, 2).to(wdtype)
        gw1 = dw1.view(C1, 1, 3, 3).to(wdtype)
        return (None, None, None, None, None, gw1, db1.to(wdtype) if db1 is not None else None, gw2, db2.to(wdtype) if db2 is not None else None,
                gw3, db3.to(wdtype) if db3 is not None else None, None, None)


def conv_subsample_packed(feats: torch.Tensor, lens_dev: torch.Tensor, pack, conv_params: List[Tuple[torch.Tensor, Optional[torch.Tensor]]],
                          time_strides: Tuple[int, int]) -> torch.Tensor:
    """
    :param feats: [B, T, F] bf16 on the device (frames beyond the lengths may hold anything)
    :param lens_dev: int32 [3, B] on the device: lengths at the input, after layer 2, after layer 3
    :param pack: PackInfo of the output frames (lengths after layer 3)
    :param conv_params: [(filter [C_out, C_in, 3, 3], bias [C_out] or None)] x 3
    :param time_strides: time strides of layers 2 and 3
    :return: packed rows [n, (F/2) * C3] bf16
    """
    (w1, b1), (w2, b2), (w3, b3) = conv_params
    return _FrontendFn.apply(feats, lens_dev, pack.row_batch, pack.row_pos, pack.cu, w1, b1, w2, b2, w3, b3, int(time_strides[0]), int(time_strides[1]))
