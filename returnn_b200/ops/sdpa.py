"""
Scaled-dot-product attention (self, causal, cross) on the tcgen05 batched GEMM with a fused mask + softmax + dropout kernel
between the two products; forward and backward.

Inputs are the usual projection outputs viewed as matrices: ``q [B, Tq, H*D]``, ``k, v [B, Tk, H*D]`` (bf16, contiguous); head
``h`` is the column block ``h*D .. (h+1)*D``, so no transposition to ``[B, H, T, D]`` is made: the batched GEMM addresses the
blocks by origin. ``k_lens`` masks padded keys, ``causal`` hides keys after the query position. The scores exist only as
``[B*H, Tq, Tk]`` buffers (padded to multiples of 64) between the kernels.

Reference semantics: returnn/frontend/_backend.py:1575-1647 (``scaled_dot_product_attention``), used by
``rf.SelfAttention``, ``rf.CausalSelfAttention``, ``rf.CrossAttention`` and the Transformer decoder.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import math
import torch
from . import _lib
from . import gemm as _gemm
from .attention_native import _bgemm
from .elementwise import _seed_tensor
from ..tensor.utils import host_to_device

_vp, _i32, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def available(x: torch.Tensor) -> bool:
    """CUDA tensor and the native library is loaded"""
    lib = _lib.get_lib()
    return x.is_cuda and lib is not None and hasattr(lib, "rb200_sdpa_softmax_fwd")


def supports(q: torch.Tensor, k: torch.Tensor, num_heads: int) -> bool:
    """shapes the kernels take: head dim a multiple of 64"""
    if not available(q) or q.dim() != 3 or k.dim() != 3:
        return False
    hd = q.shape[-1]
    if hd % num_heads:
        return False
    d = hd // num_heads
    # the contraction runs in blocks of 64 columns: a head must fill whole blocks
    return d % 64 == 0 and d <= 256 and q.shape[1] > 0 and k.shape[1] > 0


def _r64(n: int) -> int:
    return (n + 63) // 64 * 64


def _rows(t: torch.Tensor):
    """
    :param t: [B, T, H, D]
    :return: (bf16 tensor addressed in place or a contiguous copy, row pitch, head pitch) in elements. In place needs: unit stride
        over D, batch entries T rows apart, pitches that are multiples of 8 elements (16 bytes, the rule of the tensor maps), a 16-byte
        aligned start, heads inside a row.
    """
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    B, T, H, D = t.shape
    sb, st, sh, sd = t.stride()
    ok = sd == 1 and (T == 1 or st % 8 == 0) and (H == 1 or sh % 8 == 0) and t.data_ptr() % 16 == 0
    if ok and T == 1:
        st = sb if B > 1 else max((H - 1) * sh + D, 8)
        ok = st % 8 == 0
    if ok and H == 1:
        sh = D
    ok = ok and (B == 1 or sb == T * st) and sh >= D and st >= (H - 1) * sh + D
    if not ok:
        t = t.contiguous()
        return t, H * D, D
    return t, st, sh


class _SdpaFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, k_lens, H, causal, scale, p_drop):
        # q [B, Tq, H, D], k / v [B, Tk, H, D]: any views with unit stride over D whose rows and heads sit at fixed pitches, e.g. the
        # slices of a fused qkv projection; the products address them in place (row pitch = leading dimension, head pitch = column offset)
        B, Tq, _, D = q.shape
        Tk = k.shape[1]
        HD = H * D
        dev = q.device
        bf = torch.bfloat16
        q2, rq, hq = _rows(q)
        k2, rk, hk = _rows(k)
        v2, rv, hv = _rows(v)
        wq, wk, wv = (H - 1) * hq + D, (H - 1) * hk + D, (H - 1) * hv + D  # columns a row of each operand spans
        Tqp, Tkp = _r64(Tq), _r64(Tk)
        # bf16 scores (what a matmul under autocast writes) whenever a key row fits the register-resident softmax: half the traffic
        vec = Tkp <= 1024 and hasattr(_lib.get_lib(), "rb200_sdpa_softmax_fwd_bf16")
        s = torch.empty(B * H * Tqp, Tkp, dtype=bf if vec else torch.float32, device=dev)
        # 1. S = scale * Q K^T per (batch, head)
        _bgemm(q2, k2, s, m=Tq, n=Tk, k=D, a_mn=False, b_mn=False, lda=rq, ldb=rk, ldc=Tkp, a_shape=(B * Tq, wq), b_shape=(B * Tk, wk),
               offs=(Tq, 0, 0, hq, Tk, 0, 0, hk, H * Tqp * Tkp, Tqp * Tkp), batch=B * H, heads=H, lens=None, m_l=False, n_l=False, k_l=False,
               alpha=scale, out_fp32=not vec)
        # 2. P = softmax(mask(S)), Pd = dropout(P); margins up to the padded extents are written as zeros
        drop = p_drop > 0.0
        p = torch.empty(B * H * Tqp, Tkp, dtype=bf, device=dev)
        pd = torch.empty_like(p) if drop else p
        seed = _seed_tensor(dev)
        off = seed[1:2].clone()
        if drop:
            seed[1] += B * H * Tqp * Tkp
        causal_shift = Tk - Tq
        fn = _lib.bind("rb200_sdpa_softmax_fwd_bf16" if vec else "rb200_sdpa_softmax_fwd", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _vp])
        _lib.check(fn(s.data_ptr(), p.data_ptr(), pd.data_ptr() if drop else None, k_lens.data_ptr() if k_lens is not None else None, B, H, Tq, Tk,
                      Tqp, Tkp, 1 if causal else 0, causal_shift, float(p_drop), seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "sdpa_softmax_fwd")
        _lib.count_launch()
        del s
        # 3. O = Pd V
        o = torch.empty(B * Tq, HD, dtype=bf, device=dev)
        _bgemm(pd, v2, o, m=Tq, n=D, k=Tk, a_mn=False, b_mn=True, lda=Tkp, ldb=rv, ldc=HD, a_shape=(B * H * Tqp, Tkp), b_shape=(B * Tk, wv),
               offs=(H * Tqp, Tqp, 0, 0, Tk, 0, 0, hv, Tq * HD, D), batch=B * H, heads=H, lens=None, m_l=False, n_l=False, k_l=False)
        ctx.save_for_backward(q2, k2, v2, p, pd if drop else None, k_lens, off)
        ctx.geom = (B, H, Tq, Tk, D, Tqp, Tkp, bool(causal), float(scale), float(p_drop), q.dtype)
        ctx.pitches = (rq, hq, rk, hk, rv, hv)
        ctx.vec = vec
        return o.view(B, Tq, H, D).to(q.dtype)

    @staticmethod
    def backward(ctx, d_out):
        q2, k2, v2, p, pd, k_lens, off = ctx.saved_tensors
        B, H, Tq, Tk, D, Tqp, Tkp, causal, scale, p_drop, in_dtype = ctx.geom
        HD = H * D
        rq, hq, rk, hk, rv, hv = ctx.pitches
        wq, wk, wv = (H - 1) * hq + D, (H - 1) * hk + D, (H - 1) * hv + D
        dev = d_out.device
        bf = torch.bfloat16
        drop = p_drop > 0.0
        if pd is None:
            pd = p
        do2, rdo, hdo = _rows(d_out)
        wdo = (H - 1) * hdo + D
        # dV = Pd^T dO  (contraction over the query positions: rows [Tq, Tqp) of Pd are zero)
        dv = torch.empty(B * Tk, HD, dtype=bf, device=dev)
        _bgemm(pd, do2, dv, m=Tk, n=D, k=Tq, a_mn=True, b_mn=True, lda=Tkp, ldb=rdo, ldc=HD, a_shape=(B * H * Tqp, Tkp), b_shape=(B * Tq, wdo),
               offs=(H * Tqp, Tqp, 0, 0, Tq, 0, 0, hdo, Tk * HD, D), batch=B * H, heads=H, lens=None, m_l=False, n_l=False, k_l=False)
        # dPd = dO V^T
        vec = ctx.vec
        dpd = torch.empty(B * H * Tqp, Tkp, dtype=bf if vec else torch.float32, device=dev)
        _bgemm(do2, v2, dpd, m=Tq, n=Tk, k=D, a_mn=False, b_mn=False, lda=rdo, ldb=rv, ldc=Tkp, a_shape=(B * Tq, wdo), b_shape=(B * Tk, wv),
               offs=(Tq, 0, 0, hdo, Tk, 0, 0, hv, H * Tqp * Tkp, Tqp * Tkp), batch=B * H, heads=H, lens=None, m_l=False, n_l=False, k_l=False,
               out_fp32=not vec)
        ds = torch.empty(B * H * Tqp, Tkp, dtype=bf, device=dev)
        seed = _seed_tensor(dev)
        fn = _lib.bind("rb200_sdpa_softmax_bwd_bf16" if vec else "rb200_sdpa_softmax_bwd", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp, _vp])
        _lib.check(fn(p.data_ptr(), dpd.data_ptr(), ds.data_ptr(), k_lens.data_ptr() if k_lens is not None else None, B, H, Tq, Tk, Tqp, Tkp,
                      1 if causal else 0, Tk - Tq, float(p_drop), seed.data_ptr(), off.data_ptr(), _lib.stream_ptr()), "sdpa_softmax_bwd")
        _lib.count_launch()
        del dpd
        # dQ = scale * dS K ; dK = scale * dS^T Q
        dq = torch.empty(B * Tq, HD, dtype=bf, device=dev)
        _bgemm(ds, k2, dq, m=Tq, n=D, k=Tk, a_mn=False, b_mn=True, lda=Tkp, ldb=rk, ldc=HD, a_shape=(B * H * Tqp, Tkp), b_shape=(B * Tk, wk),
               offs=(H * Tqp, Tqp, 0, 0, Tk, 0, 0, hk, Tq * HD, D), batch=B * H, heads=H, lens=None, m_l=False, n_l=False, k_l=False, alpha=scale)
        dk = torch.empty(B * Tk, HD, dtype=bf, device=dev)
        _bgemm(ds, q2, dk, m=Tk, n=D, k=Tq, a_mn=True, b_mn=True, lda=Tkp, ldb=rq, ldc=HD, a_shape=(B * H * Tqp, Tkp), b_shape=(B * Tq, wq),
               offs=(H * Tqp, Tqp, 0, 0, Tq, 0, 0, hq, Tk * HD, D), batch=B * H, heads=H, lens=None, m_l=False, n_l=False, k_l=False, alpha=scale)
        return (dq.view(B, Tq, H, D).to(in_dtype), dk.view(B, Tk, H, D).to(in_dtype), dv.view(B, Tk, H, D).to(in_dtype), None, None, None, None, None)


def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, num_heads: int, k_lens: Optional[torch.Tensor] = None, causal: bool = False,
         scale: Optional[float] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """
    :param q: [B, Tq, H*D]
    :param k: [B, Tk, H*D]
    :param v: [B, Tk, H*D]
    :param k_lens: int32 [B] on the device: number of valid keys per batch entry (None: all)
    :param causal: query i sees keys j <= i + (Tk - Tq)
    :param scale: default 1/sqrt(D)
    :param dropout_p: on the attention probabilities (pass 0 outside of training)
    :return: [B, Tq, H*D], dtype of q
    """
    assert q.dim() == 3 and k.shape == v.shape and q.shape[0] == k.shape[0] and q.shape[2] == k.shape[2]
    B, Tq, HD = q.shape
    d = HD // num_heads
    o = sdpa_heads(q.unflatten(2, (num_heads, d)), k.unflatten(2, (num_heads, d)), v.unflatten(2, (num_heads, d)), k_lens=k_lens, causal=causal,
                   scale=scale, dropout_p=dropout_p)
    return o.reshape(B, Tq, HD)


def sdpa_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, k_lens: Optional[torch.Tensor] = None, causal: bool = False,
               scale: Optional[float] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """
    As :func:`sdpa` with the heads as a dim of their own: q ``[B, Tq, H, D]``, k / v ``[B, Tk, H, D]``, result ``[B, Tq, H, D]``.
    The inputs may be strided views (slices of one fused projection, heads interleaved with other columns): they are read in place.
    """
    assert q.dim() == 4 and k.shape == v.shape and q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:]
    num_heads, d = q.shape[2], q.shape[3]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if k_lens is not None:
        k_lens = host_to_device(k_lens.to(torch.int32), q.device).contiguous()
    return _SdpaFn.apply(q, k, v, k_lens, int(num_heads), bool(causal), float(scale), float(dropout_p))


def sdpa_reference(q, k, v, *, num_heads: int, k_lens=None, causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """the same in plain PyTorch fp32 (no dropout): the oracle of the tests"""
    B, Tq, HD = q.shape
    Tk = k.shape[1]
    D = HD // num_heads
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().view(B, Tq, num_heads, D).transpose(1, 2)
    kf = k.float().view(B, Tk, num_heads, D).transpose(1, 2)
    vf = v.float().view(B, Tk, num_heads, D).transpose(1, 2)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = torch.ones(B, 1, Tq, Tk, dtype=torch.bool, device=q.device)
    if k_lens is not None:
        mask = mask & (torch.arange(Tk, device=q.device)[None, None, None, :] < k_lens.to(q.device)[:, None, None, None])
    if causal:
        i = torch.arange(Tq, device=q.device)[:, None]
        j = torch.arange(Tk, device=q.device)[None, :]
        mask = mask & (j <= i + (Tk - Tq))[None, None]
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf)
    return o.transpose(1, 2).reshape(B, Tq, HD)
