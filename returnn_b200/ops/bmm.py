"""
Batched matrix product ``[Bt, M, K] x [Bt, K, N] -> [Bt, M, N]`` on the batched tcgen05 GEMM, with its own backward (two more calls of
the same kernel). This is what ``rf.matmul`` / ``rf.dot`` run on a GPU for bf16 operands (bf16 tensors, or float32 under bf16
autocast) beyond the plain ``x @ w`` case, which goes through :mod:`returnn_b200.ops.linear`.

The kernel contracts in blocks of 64. A block that reaches past the contraction extent reads zeros when the overshoot runs along the
columns of the stored operand (the tensor map fills them), but the next batch entry's rows when it runs along the rows. So the own
path is taken when every contraction that runs along rows has an extent that is a multiple of 64 (K for the product, M for the
gradient of the second operand) or there is one batch entry only; other shapes use ``torch.matmul``.

Parity: the batched case of returnn/torch/frontend/_backend.py:1677-1787 (``torch.matmul`` there).
"""

from __future__ import annotations
import torch
from . import _lib
from . import gemm as _gemm


def supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    """see the module docstring; ``a`` [Bt, M, K], ``b`` [Bt, K, N]"""
    if not (a.is_cuda and b.is_cuda and a.dim() == 3 and b.dim() == 3 and _lib.use_native(a, b) and _gemm.ENABLED):
        return False
    bf = torch.bfloat16
    autocast_bf16 = torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == bf
    if not ((a.dtype == bf and b.dtype == bf) or (autocast_bf16 and a.dtype in (bf, torch.float32) and b.dtype in (bf, torch.float32))):
        return False
    bt, m, k = a.shape
    n = b.shape[2]
    if min(bt, m, k, n) <= 0 or k % 8 or n % 8:
        return False
    return bt == 1 or (k % 64 == 0 and m % 64 == 0)


class _BmmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        from .attention_native import _bgemm

        bf = torch.bfloat16
        a2, b2 = a.to(bf).contiguous(), b.to(bf).contiguous()
        bt, m, k = a2.shape
        n = b2.shape[2]
        c = torch.empty(bt, m, n, dtype=bf, device=a.device)
        # A stored [m][k], B stored [k][n]
        _bgemm(a2, b2, c, m=m, n=n, k=k, a_mn=False, b_mn=True, lda=k, ldb=n, ldc=n, a_shape=(bt * m, k), b_shape=(bt * k, n),
               offs=(m, 0, 0, 0, k, 0, 0, 0, m * n, 0), batch=bt, heads=1, lens=None, m_l=False, n_l=False, k_l=False)
        ctx.save_for_backward(a2, b2)
        ctx.in_dtypes = (a.dtype, b.dtype)
        return c

    @staticmethod
    def backward(ctx, dc):
        from .attention_native import _bgemm

        a2, b2 = ctx.saved_tensors
        bf = torch.bfloat16
        bt, m, k = a2.shape
        n = b2.shape[2]
        dc2 = dc.to(bf).contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            # dA [m][k] = dC [m][n] . B^T: the second operand is B stored [k][n], i.e. [out column][contraction]
            da = torch.empty(bt, m, k, dtype=bf, device=dc.device)
            _bgemm(dc2, b2, da, m=m, n=k, k=n, a_mn=False, b_mn=False, lda=n, ldb=n, ldc=k, a_shape=(bt * m, n), b_shape=(bt * k, n),
                   offs=(m, 0, 0, 0, k, 0, 0, 0, m * k, 0), batch=bt, heads=1, lens=None, m_l=False, n_l=False, k_l=False)
            da = da.to(ctx.in_dtypes[0])
        if ctx.needs_input_grad[1]:
            # dB [k][n] = A^T . dC: both operands stored [contraction = m][...]
            db = torch.empty(bt, k, n, dtype=bf, device=dc.device)
            _bgemm(a2, dc2, db, m=k, n=n, k=m, a_mn=True, b_mn=True, lda=k, ldb=n, ldc=n, a_shape=(bt * m, k), b_shape=(bt * m, n),
                   offs=(m, 0, 0, 0, m, 0, 0, 0, k * n, 0), batch=bt, heads=1, lens=None, m_l=False, n_l=False, k_l=False)
            db = db.to(ctx.in_dtypes[1])
        return da, db


def bmm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """
    :param a: [Bt, M, K]
    :param b: [Bt, K, N]
    :return: [Bt, M, N]; bf16 from the own kernel where :func:`supported`, else ``torch.matmul``
    """
    if supported(a, b):
        return _BmmFn.apply(a, b)
    return torch.matmul(a, b)
