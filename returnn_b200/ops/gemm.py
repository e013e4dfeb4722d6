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
    """device word written by a kernel that gave up waiting (0 = fine)"""
    key = str(device)
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device=None):
    """raise if any GEMM launch since the last check reported a timeout (synchronises)"""
    for key, t in _status.items():
        if device is not None and key != str(device):
            continue
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError("tcgen05 GEMM reported a bounded-wait timeout: role %i, k-block %i" % (v >> 24, v & 0xFFFFFF))


def gemm(a: torch.Tensor, b: torch.Tensor, *, m: int, n: int, k: int, a_mn_major: bool, b_mn_major: bool,
         bias: Optional[torch.Tensor] = None, act: Optional[str] = None, out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, alpha: float = 1.0,
         out_act: Optional[torch.Tensor] = None, want_act_output: bool = False):
    """
    ``D[m,n] = alpha * A·B (+ bias) (act)``.

    :param a: bf16 2-D, stored ``[m, k]`` (``a_mn_major=False``) or ``[k, m]`` (True); last dim contiguous
    :param b: bf16 2-D, stored ``[n, k]`` (``b_mn_major=False``) or ``[k, n]`` (True)
    :param want_act_output: return ``(pre_activation, activated)`` instead of only the activated result
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    lda, ldb = a.stride(0), b.stride(0)
    if a.shape[0] == 1:
        lda = a.shape[1]
    if b.shape[0] == 1:
        ldb = b.shape[1]
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    c2 = None
    if want_act_output:
        c2 = out_act if out_act is not None else torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    fn = _lib.bind("rb200_gemm_bf16", [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp, _vp])
    st = status_tensor(a.device)
    _lib.check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), c2.data_ptr() if c2 is not None else None,
                  bias.data_ptr() if bias is not None else None, m, n, k, lda, ldb, out.stride(0), 1 if a_mn_major else 0,
                  1 if b_mn_major else 0, 1 if (bias is not None and bias.dtype == torch.bfloat16) else 0, _ACT[act],
                  1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0, float(alpha), st.data_ptr(), _lib.stream_ptr()), "gemm_bf16")
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
