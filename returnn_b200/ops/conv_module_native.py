"""
Binding of the fused conv-module kernels (``csrc/conv_module.cu``): GLU + depthwise conv + BatchNorm (statistics over
the valid frames) + SiLU on packed rows, forward and backward. The per-CTA partial sums of the reductions (BatchNorm
statistics, dgamma/dbeta, dfilter) live in scratch buffers allocated per call.
"""

from __future__ import annotations
import ctypes
import torch
from . import _lib

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_TT = 32


def available(x) -> bool:
    """library present with the entry points"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_glu_dwconv_fwd") and x.is_cuda and x.dtype == torch.bfloat16


def supports(channels: int, kernel: int) -> bool:
    """shapes handled: channels multiple of 64 (and 256 % (C/8) == 0 for the BN backward), up to 64 taps"""
    groups = channels // 8
    return channels % 64 == 0 and 1 <= kernel <= 64 and groups <= 256 and 256 % groups == 0


def _p(t):
    return None if t is None else t.data_ptr()


class _ConvModuleFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, filt, bias, gamma, beta, running_mean, running_var, row_batch, row_pos, lens, eps, momentum, training):
        N, C2 = x.shape
        C = C2 // 2
        K = filt.shape[-1]
        dev = x.device
        x = x.contiguous()
        f32 = filt.reshape(C, K).float().contiguous()
        b32 = bias.float().contiguous() if bias is not None else None
        g32 = gamma.float().contiguous() if gamma is not None else None
        be32 = beta.float().contiguous() if beta is not None else None
        n_tiles = (N + _TT - 1) // _TT
        y = torch.empty(N, C, dtype=torch.bfloat16, device=dev)
        part = torch.empty(n_tiles * 2 * C, dtype=torch.float32, device=dev)
        s = _lib.stream_ptr()
        fn = _lib.bind("rb200_glu_dwconv_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp])
        _lib.check(fn(x.data_ptr(), f32.data_ptr(), _p(b32), row_batch.data_ptr(), row_pos.data_ptr(), lens.data_ptr(), y.data_ptr(),
                      part.data_ptr(), N, C, K, s), "glu_dwconv_fwd")
        mean = torch.empty(C, dtype=torch.float32, device=dev)
        rstd = torch.empty(C, dtype=torch.float32, device=dev)
        if training or running_mean is None:
            fn = _lib.bind("rb200_bn_stats", [_vp, _i32, _i32, _f32, _f32, _f32, _vp, _vp, _vp, _vp, _vp])
            upd = training and running_mean is not None
            _lib.check(fn(part.data_ptr(), n_tiles, C, float(N), float(eps), float(momentum), mean.data_ptr(), rstd.data_ptr(),
                          running_mean.data_ptr() if upd else None, running_var.data_ptr() if upd else None, s), "bn_stats")
            _lib.count_launch()
        else:
            mean.copy_(running_mean.float())
            rstd.copy_(torch.rsqrt(running_var.float() + eps))
        z = torch.empty(N, C, dtype=torch.bfloat16, device=dev)
        fn = _lib.bind("rb200_bn_silu_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp])
        _lib.check(fn(y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), _p(g32), _p(be32), z.data_ptr(), N, C, s), "bn_silu_fwd")
        _lib.count_launch(2)
        ctx.save_for_backward(x, f32, y, mean, rstd, g32, be32, row_batch, row_pos, lens)
        ctx.meta = (N, C, K, training, bias is not None, gamma is not None, beta is not None, filt.shape, filt.dtype,
                    bias.dtype if bias is not None else None, gamma.dtype if gamma is not None else None, beta.dtype if beta is not None else None)
        return z

    @staticmethod
    def backward(ctx, dz):
        x, f32, y, mean, rstd, g32, be32, row_batch, row_pos, lens = ctx.saved_tensors
        N, C, K, training, has_bias, has_gamma, has_beta, fshape, fdtype, bdtype, gdtype, bedtype = ctx.meta
        dev = dz.device
        dz = dz.contiguous()
        s = _lib.stream_ptr()
        n_tiles_a = min(592, max(1, (N + 15) // 16))
        ds = torch.empty(N, C, dtype=torch.bfloat16, device=dev)
        part_a = torch.empty(n_tiles_a * 2 * C, dtype=torch.float32, device=dev)
        sum_ds = torch.empty(C, dtype=torch.float32, device=dev)
        sum_ds_yh = torch.empty(C, dtype=torch.float32, device=dev)
        fn = _lib.bind("rb200_bn_silu_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i64, _i32, _i32, _vp])
        _lib.check(fn(y.data_ptr(), dz.data_ptr(), mean.data_ptr(), rstd.data_ptr(), _p(g32), _p(be32), ds.data_ptr(), part_a.data_ptr(),
                      n_tiles_a, sum_ds.data_ptr(), sum_ds_yh.data_ptr(), N, C, 1 if training else 0, s), "bn_silu_bwd")
        _lib.count_launch(3 if training else 2)
        if not training:
            # eval statistics are constants: dy = gamma * rstd * ds
            scale = rstd * (g32 if g32 is not None else 1.0)
            ds = (ds.float() * scale).to(torch.bfloat16)
        n_tiles = (N + _TT - 1) // _TT
        dx = torch.empty_like(x)
        part = torch.empty(n_tiles * C * (K + 1), dtype=torch.float32, device=dev)
        dfilt = torch.empty(C, K, dtype=torch.float32, device=dev)
        dbias = torch.empty(C, dtype=torch.float32, device=dev)
        fn = _lib.bind("rb200_glu_dwconv_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp])
        _lib.check(fn(x.data_ptr(), ds.data_ptr(), f32.data_ptr(), row_batch.data_ptr(), row_pos.data_ptr(), lens.data_ptr(), dx.data_ptr(),
                      part.data_ptr(), dfilt.data_ptr(), dbias.data_ptr(), N, C, K, s), "glu_dwconv_bwd")
        _lib.count_launch(2)
        return (dx, dfilt.reshape(fshape).to(fdtype), dbias.to(bdtype) if has_bias else None,
                sum_ds_yh.to(gdtype) if has_gamma else None, sum_ds.to(bedtype) if has_beta else None,
                None, None, None, None, None, None, None, None)


def glu_dwconv_bn_silu(x, filt, bias, bn, pack, *, training):
    """fused path; ``bn`` is the rf.BatchNorm module (its running statistics are updated in place in training)"""
    gamma = bn.gamma.raw_tensor if bn.affine else None
    beta = bn.beta.raw_tensor if bn.affine else None
    rm = bn.running_mean.raw_tensor if bn.running_mean is not None else None
    rv = bn.running_variance.raw_tensor if bn.running_variance is not None else None
    return _ConvModuleFn.apply(x, filt, bias, gamma, beta, rm, rv, pack.row_batch, pack.row_pos, pack.lens, float(bn.eps), float(bn.momentum), bool(training))
