"""
Relative-position self-attention on packed rows, B200 path.

Stages (forward): ``att_prepare`` (packed qkv -> zero-padded Qu = q+u, Qv = q+v, K, V) -> batched tcgen05 GEMMs
``S_ac = scale * Qu K^T`` and ``G = scale * Qv P^T`` (fp32 out) -> ``att_softmax_fwd`` (shifted bias as an index into G,
key-length mask, softmax, dropout) -> batched GEMM ``O = Wd V`` -> gather back to packed rows.
Backward: ``dWd = dO V^T``, ``dV = Wd^T dO``, ``att_softmax_bwd`` (exact delta, un-shift into dG), ``dQu = dS K``,
``dK = dS^T Qu``, ``dQv = dG P``, ``dP = sum_b dG^T Qv`` (one GEMM per head over all rows), then one pack kernel.

Buffers per call: padded operands ``[B*Lp, H*D]``, scores ``[B*H*Lp, Lp]`` and bias band ``[H, B, Lp, Rp]`` with
``Lp`` = longest sequence rounded up to 64 and ``Rp = 2*Lp``. Limits: ``Lp <= 512``, ``D % 64 == 0``.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import torch
from . import _lib
from . import gemm as _gemm
from .elementwise import _seed_tensor

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
MAX_LEN = 512


def available(*tensors) -> bool:
    """library present with the attention entry points, bf16 inputs"""
    lib = _lib.get_lib()
    if lib is None or not hasattr(lib, "rb200_att_softmax_fwd") or not hasattr(lib, "rb200_gemm_bf16_batched"):
        return False
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors) and _gemm.ENABLED


def supports_sdpa(q, k, v, causal: bool) -> bool:
    """``[B, H, T, D]`` operands (bf16 or under bf16 autocast) with a head dim that fills the 64-wide contraction blocks"""
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape or q.shape[:2] != k.shape[:2] or q.shape[-1] != k.shape[-1]:
        return False
    if q.dtype != torch.bfloat16 and not (q.dtype == torch.float32 and torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.bfloat16):
        return False
    d = q.shape[-1]
    return d % 64 == 0 and d <= 256 and q.shape[2] > 0 and k.shape[2] > 0


def supports_rel_pos(q, k, v, pos) -> bool:
    """padded [N,H,T,D] entry: routed through the packed kernel by the caller when possible"""
    return False


def supports_packed(num_heads: int, head_dim: int, max_len: int) -> bool:
    """shapes handled by the packed rel-pos path"""
    # head_dim must fill whole 64-wide K tiles: a narrower head would pull the neighbouring head into the contraction
    return head_dim % 64 == 0 and 0 < max_len <= MAX_LEN


def _bgemm(a, b, c, *, m, n, k, a_mn, b_mn, lda, ldb, ldc, a_shape, b_shape, offs, batch, heads, lens, m_l, n_l, k_l, alpha=1.0,
           out_fp32=False):
    fn = _lib.bind("rb200_gemm_bf16_batched", [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                               _i32, _i32, _i32, _i32, _f32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _vp])
    arr = (ctypes.c_longlong * 10)(*offs)
    st = _gemm.status_tensor(a.device)
    _lib.check(fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, a_shape[0], a_shape[1], b_shape[0], b_shape[1], lda, ldb, ldc, m, n, k,
                  1 if a_mn else 0, 1 if b_mn else 0, 0, 0, 1 if out_fp32 else 0, 0, float(alpha), batch, heads, ctypes.addressof(arr),
                  lens.data_ptr() if lens is not None else None, 1 if m_l else 0, 1 if n_l else 0, 1 if k_l else 0, st.data_ptr(),
                  _lib.stream_ptr()), "gemm_bf16_batched")
    _lib.count_launch()


class _RelPosAttPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, u, v, row_batch, row_pos, lens, B, H, D, max_len, scale, p_drop):
        dev = qkv.device
        N = qkv.shape[0]
        HD = H * D
        Lp = (max_len + 63) // 64 * 64
        Rp = 2 * Lp
        R = pos.shape[0]
        center = (R - 1) // 2
        assert R <= Rp and center >= max_len - 1
        qkv = qkv.contiguous()
        pos = pos.contiguous()
        uf = u.float().contiguous() if u is not None else None
        vf = v.float().contiguous() if v is not None else None
        bf = torch.bfloat16
        qu = torch.zeros(B * Lp, HD, dtype=bf, device=dev)
        qv = torch.zeros(B * Lp, HD, dtype=bf, device=dev)
        kk = torch.zeros(B * Lp, HD, dtype=bf, device=dev)
        vv = torch.zeros(B * Lp, HD, dtype=bf, device=dev)
        fn = _lib.bind("rb200_att_prepare", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp])
        _lib.check(fn(qkv.data_ptr(), uf.data_ptr() if uf is not None else None, vf.data_ptr() if vf is not None else None,
                      row_batch.data_ptr(), row_pos.data_ptr(), qu.data_ptr(), qv.data_ptr(), kk.data_ptr(), vv.data_ptr(), N, H, D, Lp,
                      _lib.stream_ptr()), "att_prepare")
        _lib.count_launch()
        # P padded to Rp rows so that tile reads stay inside the tensor
        pos_p = pos
        s_ac = torch.empty(B * H * Lp, Lp, dtype=torch.float32, device=dev)
        g = torch.empty(H * B * Lp, Rp, dtype=torch.float32, device=dev)
        # 1. S_ac = scale * Qu K^T
        _bgemm(qu, kk, s_ac, m=Lp, n=Lp, k=D, a_mn=False, b_mn=False, lda=HD, ldb=HD, ldc=Lp, a_shape=(B * Lp, HD), b_shape=(B * Lp, HD),
               offs=(Lp, 0, 0, D, Lp, 0, 0, D, H * Lp * Lp, Lp * Lp), batch=B * H, heads=H, lens=lens, m_l=True, n_l=True, k_l=False,
               alpha=scale, out_fp32=True)
        # 2. G = scale * Qv P^T, stored [H, B, Lp, Rp]
        _bgemm(qv, pos_p, g, m=Lp, n=R, k=D, a_mn=False, b_mn=False, lda=HD, ldb=HD, ldc=Rp, a_shape=(B * Lp, HD), b_shape=(R, HD),
               offs=(Lp, 0, 0, D, 0, 0, 0, D, Lp * Rp, B * Lp * Rp), batch=B * H, heads=H, lens=lens, m_l=True, n_l=False, k_l=False,
               alpha=scale, out_fp32=True)
        w = torch.zeros(B * H * Lp, Lp, dtype=bf, device=dev)
        drop = p_drop > 0.0
        wd = torch.zeros(B * H * Lp, Lp, dtype=bf, device=dev) if drop else w
        seed = _seed_tensor(dev)
        off = seed[1:2].clone()
        if drop:
            seed[1] += B * H * Lp * Lp
        fn = _lib.bind("rb200_att_softmax_fwd", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _vp])
        _lib.check(fn(s_ac.data_ptr(), g.data_ptr(), w.data_ptr(), wd.data_ptr(), lens.data_ptr(), B, H, Lp, Rp, center, float(p_drop),
                      seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "att_softmax_fwd")
        _lib.count_launch()
        del s_ac, g
        # 3. O = Wd V
        o_pad = torch.empty(B * Lp, HD, dtype=bf, device=dev)
        _bgemm(wd, vv, o_pad, m=Lp, n=D, k=Lp, a_mn=False, b_mn=True, lda=Lp, ldb=HD, ldc=HD, a_shape=(B * H * Lp, Lp), b_shape=(B * Lp, HD),
               offs=(H * Lp, Lp, 0, 0, Lp, 0, 0, D, Lp * HD, D), batch=B * H, heads=H, lens=lens, m_l=True, n_l=False, k_l=True)
        out = torch.empty(N, HD, dtype=bf, device=dev)
        gfn = _lib.bind("rb200_att_rows_gather", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp])
        _lib.check(gfn(o_pad.data_ptr(), out.data_ptr(), row_batch.data_ptr(), row_pos.data_ptr(), N, HD, Lp, 0, _lib.stream_ptr()), "att_gather")
        _lib.count_launch()
        ctx.save_for_backward(qu, qv, kk, vv, w, pos_p, row_batch, row_pos, lens, off)
        ctx.dims = (B, H, D, Lp, Rp, R, center, N, scale, p_drop)
        ctx.u_dtype = u.dtype if u is not None else None
        ctx.v_dtype = v.dtype if v is not None else None
        return out

    @staticmethod
    def backward(ctx, d_out):
        qu, qv, kk, vv, w, pos_p, row_batch, row_pos, lens, off = ctx.saved_tensors
        B, H, D, Lp, Rp, R, center, N, scale, p_drop = ctx.dims
        dev = d_out.device
        HD = H * D
        bf = torch.bfloat16
        d_out = d_out.contiguous()
        do_pad = torch.zeros(B * Lp, HD, dtype=bf, device=dev)
        gfn = _lib.bind("rb200_att_rows_gather", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp])
        _lib.check(gfn(d_out.data_ptr(), do_pad.data_ptr(), row_batch.data_ptr(), row_pos.data_ptr(), N, HD, Lp, 1, _lib.stream_ptr()), "att_scatter")
        _lib.count_launch()
        drop = p_drop > 0.0
        seed = _seed_tensor(dev)
        if drop:
            # re-create the dropped probabilities (same counter-based mask as in forward)
            wd = torch.zeros_like(w)
            fn = _lib.bind("rb200_att_redrop", [_vp, _vp, _vp, _i32, _i32, _i32, _f32, _vp, _vp, _vp])
            _lib.check(fn(w.data_ptr(), wd.data_ptr(), lens.data_ptr(), B, H, Lp, float(p_drop), seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "att_redrop")
            _lib.count_launch()
        else:
            wd = w
        # 4. dWd = dO V^T
        dwd = torch.empty(B * H * Lp, Lp, dtype=torch.float32, device=dev)
        _bgemm(do_pad, vv, dwd, m=Lp, n=Lp, k=D, a_mn=False, b_mn=False, lda=HD, ldb=HD, ldc=Lp, a_shape=(B * Lp, HD), b_shape=(B * Lp, HD),
               offs=(Lp, 0, 0, D, Lp, 0, 0, D, H * Lp * Lp, Lp * Lp), batch=B * H, heads=H, lens=lens, m_l=True, n_l=True, k_l=False, out_fp32=True)
        # 5. dV = Wd^T dO
        dv_pad = torch.empty(B * Lp, HD, dtype=bf, device=dev)
        _bgemm(wd, do_pad, dv_pad, m=Lp, n=D, k=Lp, a_mn=True, b_mn=True, lda=Lp, ldb=HD, ldc=HD, a_shape=(B * H * Lp, Lp), b_shape=(B * Lp, HD),
               offs=(H * Lp, Lp, 0, 0, Lp, 0, 0, D, Lp * HD, D), batch=B * H, heads=H, lens=lens, m_l=True, n_l=False, k_l=True)
        ds = torch.zeros(B * H * Lp, Lp, dtype=bf, device=dev)
        dg = torch.zeros(H * B * Lp, Rp, dtype=bf, device=dev)
        fn = _lib.bind("rb200_att_softmax_bwd", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _vp])
        _lib.check(fn(w.data_ptr(), dwd.data_ptr(), ds.data_ptr(), dg.data_ptr(), lens.data_ptr(), B, H, Lp, Rp, center, float(p_drop),
                      seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "att_softmax_bwd")
        _lib.count_launch()
        del dwd
        # 6. dQu = scale * dS K
        dqu = torch.zeros(B * Lp, HD, dtype=bf, device=dev)  # zero tails: the column sums below run over all rows
        _bgemm(ds, kk, dqu, m=Lp, n=D, k=Lp, a_mn=False, b_mn=True, lda=Lp, ldb=HD, ldc=HD, a_shape=(B * H * Lp, Lp), b_shape=(B * Lp, HD),
               offs=(H * Lp, Lp, 0, 0, Lp, 0, 0, D, Lp * HD, D), batch=B * H, heads=H, lens=lens, m_l=True, n_l=False, k_l=True, alpha=scale)
        # 7. dK = scale * dS^T Qu
        dk_pad = torch.empty(B * Lp, HD, dtype=bf, device=dev)
        _bgemm(ds, qu, dk_pad, m=Lp, n=D, k=Lp, a_mn=True, b_mn=True, lda=Lp, ldb=HD, ldc=HD, a_shape=(B * H * Lp, Lp), b_shape=(B * Lp, HD),
               offs=(H * Lp, Lp, 0, 0, Lp, 0, 0, D, Lp * HD, D), batch=B * H, heads=H, lens=lens, m_l=True, n_l=False, k_l=True, alpha=scale)
        # 8. dQv = scale * dG P
        dqv = torch.zeros(B * Lp, HD, dtype=bf, device=dev)
        _bgemm(dg, pos_p, dqv, m=Lp, n=D, k=R, a_mn=False, b_mn=True, lda=Rp, ldb=HD, ldc=HD, a_shape=(H * B * Lp, Rp), b_shape=(R, HD),
               offs=(Lp, B * Lp, 0, 0, 0, 0, 0, D, Lp * HD, D), batch=B * H, heads=H, lens=lens, m_l=True, n_l=False, k_l=False, alpha=scale)
        # 9. dP[h] = scale * dG[h]^T Qv[h] over all rows of all sequences
        dpos = torch.empty(R, HD, dtype=bf, device=dev)
        _bgemm(dg, qv, dpos, m=R, n=D, k=B * Lp, a_mn=True, b_mn=True, lda=Rp, ldb=HD, ldc=HD, a_shape=(H * B * Lp, Rp), b_shape=(B * Lp, HD),
               offs=(0, B * Lp, 0, 0, 0, 0, 0, D, 0, D), batch=H, heads=H, lens=None, m_l=False, n_l=False, k_l=False, alpha=scale)
        dqkv = torch.empty(N, 3 * HD, dtype=bf, device=dev)
        pfn = _lib.bind("rb200_att_pack_dqkv", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp])
        _lib.check(pfn(dqu.data_ptr(), dqv.data_ptr(), dk_pad.data_ptr(), dv_pad.data_ptr(), row_batch.data_ptr(), row_pos.data_ptr(),
                       dqkv.data_ptr(), N, H, D, Lp, _lib.stream_ptr()), "att_pack_dqkv")
        _lib.count_launch()
        du = dqu.float().sum(dim=0).reshape(H, D).to(ctx.u_dtype) if ctx.u_dtype is not None else None
        dvb = dqv.float().sum(dim=0).reshape(H, D).to(ctx.v_dtype) if ctx.v_dtype is not None else None
        return dqkv, dpos, du, dvb, None, None, None, None, None, None, None, None, None


def rel_pos_attention_packed(qkv, pos, u, v, pack, *, num_heads: int, head_dim: int, scale: float, dropout_p: float = 0.0):
    """
    :param qkv: [N, H*3*D] bf16, per head grouped (q, k, v)
    :param pos: [2*L-1, H*D] bf16 projected relative position embeddings, row r = distance r-(L-1), L >= pack.max_len
    :param u, v: [H, D] biases (any float dtype) or None
    :return: [N, H*D] bf16
    """
    return _RelPosAttPacked.apply(qkv, pos.to(torch.bfloat16), u, v, pack.row_batch, pack.row_pos, pack.lens, pack.batch, num_heads,
                                  head_dim, pack.max_len, float(scale), float(dropout_p))


def sdpa(q, k, v, *, kv_lens, scale, causal, dropout_p):
    """``[B, H, T, D]`` layout of the RF attention functions -> the ``[B, T, H*D]`` kernels of :mod:`returnn_b200.ops.sdpa`"""
    from . import sdpa as _sdpa

    lens = None
    if kv_lens is not None:
        lens = kv_lens
        while lens.dim() > 1:  # given per (batch, head): the heads share the lengths
            lens = lens[..., 0]
    # [B, T, H, D] views of the same memory: the kernels take row and head pitches, so the slices of a fused projection are not copied
    o = _sdpa.sdpa_heads(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), k_lens=lens, causal=causal, scale=scale, dropout_p=dropout_p)
    return o.transpose(1, 2)


def rel_pos_attention(q, k, v, pos, u, vb, lens, *, scale, dropout_p):
    """not built (the packed entry is the B200 path)"""
    raise NotImplementedError
