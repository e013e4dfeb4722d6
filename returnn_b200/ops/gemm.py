"""
bf16 GEMM on 5th-gen tensor cores (``csrc/gemm_tcgen05.cu``): TMA-fed shared-memory ring, ``tcgen05.mma`` issued by one
thread into a TMEM accumulator, epilogue warps read TMEM with ``tcgen05.ld`` and apply bias / activation.

``gemm`` is the raw entry (row-major operands, optional transposes expressed as operand "major-ness", so no transposed
copies are ever made); ``linear_bf16`` is the autograd function behind :func:`returnn_b200.ops.linear.linear`:
forward ``X·W + b`` (+activation), backward ``dX = dY·W^T`` and ``dW = X^T·dY`` on the same kernel.
"""

from __future__ import annotations
from typing import Dict, Optional
import ctypes
import os
import torch
from . import _lib
from . import status as _status_board

_vp, _i32, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
ENABLED = os.environ.get("RETURNN_B200_GEMM", "1") == "1"
_ACT = {None: 0, "relu": 1, "silu": 2, "swish": 2, "gelu": 3}
_status: Dict[str, torch.Tensor] = {}


def available(x: torch.Tensor) -> bool:
    """library present with the GEMM entry point"""
    if not x.is_cuda:
        return False
    if not _lib.use_native(x):
        return False
    return hasattr(_lib.get_lib(), "rb200_gemm_bf16")


def status_tensor(device) -> torch.Tensor:
    """
    Device word written by a kernel that gave up waiting (0 = fine): the GEMM slot of the device's status board
    (:mod:`returnn_b200.ops.status`), which the training loop reads once per step.
    """
    t = _status.get(device)
    if t is None:
        t = _status_board.word(device, _status_board.SLOT_GEMM)
        _status[device] = t
    return t


def check_status(device=None):
    """raise ``KernelWaitTimeout`` if any kernel since the last check reported a timeout (synchronises)"""
    _status_board.check_now(device)


KERNEL = os.environ.get("RETURNN_B200_GEMM_KERNEL", "persistent")  # "persistent" | "legacy" (one tile per CTA, plain epilogue)
_u64 = ctypes.c_ulonglong


def gemm(a: torch.Tensor, b: torch.Tensor, *, m: int, n: int, k: int, a_mn_major: bool, b_mn_major: bool,
         bias: Optional[torch.Tensor] = None, act: Optional[str] = None, out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, alpha: float = 1.0,
         out_act: Optional[torch.Tensor] = None, want_act_output: bool = False,
         dact_z: Optional[torch.Tensor] = None, dropout_p: float = 0.0, dropout_seed: Optional[torch.Tensor] = None,
         dropout_offset: Optional[torch.Tensor] = None, dropout_site: int = 0,
         resid: Optional[torch.Tensor] = None, res_scale: float = 1.0, atomic: bool = False, split_k: int = 0):
    """
    ``D[m,n] = epilogue(alpha * A·B)``; epilogue order: ``+ bias``, ``* act'(dact_z)`` or ``act``, dropout, ``resid + res_scale *``.

    :param a: bf16 2-D, stored ``[m, k]`` (``a_mn_major=False``) or ``[k, m]`` (True); last dim contiguous
    :param b: bf16 2-D, stored ``[n, k]`` (``b_mn_major=False``) or ``[k, n]`` (True)
    :param want_act_output: return ``(pre_activation, final)`` instead of only the final result
    :param dact_z: bf16 ``[m, n]`` (same pitch as out): multiply by the derivative of ``act`` at ``dact_z`` (nothing is activated then)
    :param dropout_p: drop the (activated) value with a counter-based mask: element ``(r, c)`` uses counter
        ``dropout_offset[0] + dropout_site + r*pitch + c`` under key ``dropout_seed[0]`` (int64 device tensors)
    :param resid: bf16 ``[m, n]``: ``resid + res_scale * value``
    :param atomic: fp32 out only: add into ``out`` with atomics; the contraction may then be split over CTAs (``split_k``, 0 = auto)
    """
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16) and a.dim() == 2 and b.dim() == 2
    fp16 = a.dtype == torch.float16  # fp16 operands (3 more mantissa bits, smaller range): same kernels, other MMA operand format
    assert a.stride(1) == 1 and b.stride(1) == 1
    lda, ldb = a.stride(0), b.stride(0)
    if a.shape[0] == 1:
        lda = a.shape[1]
    if b.shape[0] == 1:
        ldb = b.shape[1]
    if out is None:
        assert not atomic
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    c2 = None
    if want_act_output:
        c2 = out_act if out_act is not None else torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    st = status_tensor(a.device)
    extended = dact_z is not None or dropout_p > 0.0 or resid is not None or atomic or fp16
    bias_bf16 = 1 if (bias is not None and bias.dtype == torch.bfloat16) else 0
    if KERNEL == "legacy" and not extended:
        fn = _lib.bind("rb200_gemm_bf16", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp])
        _lib.check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), c2.data_ptr() if c2 is not None else None,
                      bias.data_ptr() if bias is not None else None, m, n, k, lda, ldb, out.stride(0), 1 if a_mn_major else 0,
                      1 if b_mn_major else 0, bias_bf16, _ACT[act],
                      1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0, float(alpha), st.data_ptr(), _lib.stream_ptr()), "gemm_bf16")
    else:
        for t in (dact_z, resid):
            assert t is None or (t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.stride(0) == out.stride(0))
        fn = _lib.bind("rb200_gemm_fp16_ex" if fp16 else "rb200_gemm_bf16_ex", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32,
                                              _vp, _f32, _vp, _vp, _u64, _vp, _f32, _i32, _vp, _vp])
        _lib.check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), c2.data_ptr() if c2 is not None else None,
                      bias.data_ptr() if bias is not None else None, m, n, k, lda, ldb, out.stride(0), 1 if a_mn_major else 0,
                      1 if b_mn_major else 0, bias_bf16, _ACT[act], 1 if out.dtype == torch.float32 else 0,
                      2 if atomic else (1 if accumulate else 0), float(alpha),
                      dact_z.data_ptr() if dact_z is not None else None, float(dropout_p),
                      dropout_seed.data_ptr() if dropout_seed is not None else None,
                      dropout_offset.data_ptr() if dropout_offset is not None else None, int(dropout_site),
                      resid.data_ptr() if resid is not None else None, float(res_scale), int(split_k), st.data_ptr(), _lib.stream_ptr()),
                   "gemm_bf16_ex")
    _lib.count_launch()
    if want_act_output:
        return out, c2
    return out


def _ok_operand(t: torch.Tensor) -> bool:
    return t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and (t.dim() < 2 or t.stride(0) % 8 == 0 or t.shape[0] == 1)


def _act_grad(z: torch.Tensor, dy: torch.Tensor, act: str) -> torch.Tensor:
    zf = z.float()
    if act == "relu":
        return (dy.float() * (zf > 0)).to(dy.dtype)
    if act in ("silu", "swish"):
        s = torch.sigmoid(zf)
        return (dy.float() * (s * (1 + zf * (1 - s)))).to(dy.dtype)
    if act == "gelu":
        cdf = 0.5 * (1 + torch.erf(zf * 0.7071067811865476))
        pdf = torch.exp(-0.5 * zf * zf) * 0.3989422804014327
        return (dy.float() * (cdf + zf * pdf)).to(dy.dtype)
    raise ValueError(act)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w, bias, act):
        m, k = x2.shape
        n = w.shape[1]
        need_z = act is not None and (x2.requires_grad or w.requires_grad)
        if need_z:
            z, y = gemm(x2, w, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, bias=bias, act=act, want_act_output=True)
        else:
            z, y = None, gemm(x2, w, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, bias=bias, act=act)
        ctx.save_for_backward(x2, w, z)
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w, z = ctx.saved_tensors
        m, k = x2.shape
        n = w.shape[1]
        dy = dy.contiguous()
        if ctx.act is not None:
            dy = _act_grad(z, dy, ctx.act)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dX[m,k] = dY[m,n] · W[k,n]^T : contraction over n, W rows are contiguous in n -> "K-major" B
            dx = gemm(dy, w, m=m, n=k, k=n, a_mn_major=False, b_mn_major=False)
        if ctx.needs_input_grad[1]:
            # dW[k,n] = X[m,k]^T · dY[m,n] : contraction over m, both operands contiguous in their output dim
            dw = gemm(x2, dy, m=k, n=n, k=m, a_mn_major=True, b_mn_major=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(dim=0).to(ctx.bias_dtype)
        return dx, dw, db, None


class _ArenaLinearFn(torch.autograd.Function):
    """
    Linear layer whose weight lives in a parameter arena: the forward reads the bf16 copy of the weight, the backward adds the
    weight / bias gradients straight into the fp32 gradient arena (split-K GEMM with atomics, column-sum kernel) and returns
    only the input gradient, so no gradient tensors are created and nothing is cast.
    """

    @staticmethod
    def forward(ctx, x2, w16, bias32, gw32, gb32, act):
        m, k = x2.shape
        n = w16.shape[1]
        if act is not None:
            z, y = gemm(x2, w16, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, bias=bias32, act=act, want_act_output=True)
        else:
            z, y = None, gemm(x2, w16, m=m, n=n, k=k, a_mn_major=False, b_mn_major=True, bias=bias32)
        ctx.save_for_backward(x2, w16, z)
        ctx.act, ctx.gw32, ctx.gb32 = act, gw32, gb32
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w16, z = ctx.saved_tensors
        m, k = x2.shape
        n = w16.shape[1]
        dy = dy.contiguous()
        if ctx.act is not None:
            dy = _act_grad(z, dy, ctx.act)
        dx = gemm(dy, w16, m=m, n=k, k=n, a_mn_major=False, b_mn_major=False) if ctx.needs_input_grad[0] else None
        if ctx.gw32 is not None:
            gemm(x2, dy, m=k, n=n, k=m, a_mn_major=True, b_mn_major=True, out=ctx.gw32, atomic=True)
        if ctx.gb32 is not None:
            fn = _lib.bind("rb200_colsum_bf16", [_vp, _vp, _i32, _i32, _vp])
            _lib.check(fn(dy.data_ptr(), ctx.gb32.data_ptr(), m, n, _lib.stream_ptr()), "colsum")
            _lib.count_launch()
        from ..parallel import grad_reducer as _gr

        _gr.notify_grads_written([ctx.gw32, ctx.gb32])
        return dx, None, None, None, None, None


def linear_arena(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation: Optional[str], arena) -> Optional[torch.Tensor]:
    """
    ``x @ weight (+ bias)`` for fp32 parameters that live in ``arena`` (a :class:`returnn_b200.parallel.arena.ParamArena`
    with fp32 gradients); returns None when this path does not apply (caller falls back to :func:`linear_bf16`).
    The parameter gradients do not pass through autograd: they are accumulated into ``arena.flat_grad``.
    """
    if arena is None or not x.requires_grad or weight.dtype != torch.float32 or arena.grad_dtype != torch.float32 or weight.dim() != 2:
        return None
    if not available(x) or not weight.is_contiguous() or weight.shape[0] % 8 or weight.shape[1] % 8:
        return None

    def _views(p):
        off = (p.data_ptr() - arena.flat_param.data_ptr()) // 4
        if not (0 <= off < arena.total):
            return None, None
        sh = arena.shadow_bf16()[off: off + p.numel()].view(p.shape)
        g = arena.flat_grad[off: off + p.numel()].view(p.shape) if p.requires_grad else None
        return sh, g

    w16, gw = _views(weight)
    if w16 is None:
        return None
    gb = None
    if bias is not None:
        if bias.dtype != torch.float32:
            return None
        _, gb = _views(bias)
        if gb is None and bias.requires_grad:
            return None
    arena.sync_shadow()
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _ArenaLinearFn.apply(x2, w16, bias, gw, gb, activation)
    return y.reshape(*x.shape[:-1], w16.shape[1])


class _PaddedOutLinearFn(torch.autograd.Function):
    """see :func:`linear_arena_padded_out`"""

    @staticmethod
    def forward(ctx, x2, w_pad, bias_pad, gw32, gb32, n):
        m, k = x2.shape
        n_pad = w_pad.shape[1]
        y = gemm(x2, w_pad, m=m, n=n_pad, k=k, a_mn_major=False, b_mn_major=True, bias=bias_pad)
        ctx.save_for_backward(x2, w_pad)
        ctx.gw32, ctx.gb32, ctx.n = gw32, gb32, n
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w_pad = ctx.saved_tensors
        m, k = x2.shape
        n_pad, n = w_pad.shape[1], ctx.n
        dy = dy.contiguous()
        dx = gemm(dy, w_pad, m=m, n=k, k=n_pad, a_mn_major=False, b_mn_major=False) if ctx.needs_input_grad[0] else None
        if ctx.gw32 is not None:
            # only the first n columns of dy reach the parameter gradient [k, n] (its pitch n is not a multiple of 8: scalar atomics)
            gemm(x2, dy, m=k, n=n, k=m, a_mn_major=True, b_mn_major=True, out=ctx.gw32, atomic=True)
        if ctx.gb32 is not None:
            tmp = torch.zeros(n_pad, dtype=torch.float32, device=dy.device)
            fn = _lib.bind("rb200_colsum_bf16", [_vp, _vp, _i32, _i32, _vp])
            _lib.check(fn(dy.data_ptr(), tmp.data_ptr(), m, n_pad, _lib.stream_ptr()), "colsum")
            _lib.count_launch()
            ctx.gb32.add_(tmp[:n])
        from ..parallel import grad_reducer as _gr

        _gr.notify_grads_written([ctx.gw32, ctx.gb32])
        return dx, None, None, None, None, None


_padded_cache = {}


def linear_arena_padded_out(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], arena, *, pad_bias: float = -1e30) -> Optional[torch.Tensor]:
    """
    Output layer whose width ``n`` is not a multiple of 8 (e.g. a vocabulary of 10000 + blank): TMA needs row pitches of 16
    bytes, so the layer is computed ``n_pad = ceil8(n)`` wide. The extra columns have zero weights and bias ``pad_bias``: with
    the default they are classes of probability exactly 0 under a following (log-)softmax, receive gradient 0 and change
    nothing; the caller treats the result as ``n_pad`` classes.

    :return: ``[..., n_pad]`` bf16, or None when the arena path does not apply (see :func:`linear_arena`)
    """
    if arena is None or not x.requires_grad or weight.dtype != torch.float32 or arena.grad_dtype != torch.float32 or weight.dim() != 2:
        return None
    k, n = weight.shape
    if not available(x) or not weight.is_contiguous() or k % 8 or n % 8 == 0:
        return None
    off = (weight.data_ptr() - arena.flat_param.data_ptr()) // 4
    if not (0 <= off < arena.total):
        return None
    n_pad = (n + 7) // 8 * 8
    arena.sync_shadow()
    w16 = arena.shadow_bf16()[off: off + weight.numel()].view(k, n)
    gw = arena.flat_grad[off: off + weight.numel()].view(k, n) if weight.requires_grad else None
    gb = None
    key = (weight.data_ptr(), n_pad, str(x.device))
    bufs = _padded_cache.get(key)
    if bufs is None:
        bufs = (torch.zeros(k, n_pad, dtype=torch.bfloat16, device=x.device), torch.full((n_pad,), pad_bias, dtype=torch.float32, device=x.device))
        _padded_cache[key] = bufs
    w_pad, bias_pad = bufs
    w_pad[:, :n].copy_(w16)
    if bias is not None:
        if bias.dtype != torch.float32:
            return None
        boff = (bias.data_ptr() - arena.flat_param.data_ptr()) // 4
        if bias.requires_grad:
            if not (0 <= boff < arena.total):
                return None
            gb = arena.flat_grad[boff: boff + n]
        bias_pad[:n].copy_(bias.detach())
    else:
        bias_pad[:n].zero_()
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _PaddedOutLinearFn.apply(x2, w_pad, bias_pad, gw, gb, n)
    return y.reshape(*x.shape[:-1], n_pad)


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation: Optional[str]) -> torch.Tensor:
    """``x[..., in] @ weight[in, out] (+ bias) (activation)`` with bf16 operands"""
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    w = weight if weight.dtype == torch.bfloat16 else weight.to(torch.bfloat16)
    if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
        bias = bias.float()
    if not w.is_contiguous():
        w = w.contiguous()
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _LinearFn.apply(x2, w, bias, activation)
    return y.reshape(*x.shape[:-1], w.shape[1])
