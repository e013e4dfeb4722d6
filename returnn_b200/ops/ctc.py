"""
CTC loss with fused log-softmax.

``ctc_loss`` takes padded logits ``[B, T, V]``; ``ctc_loss_packed`` takes packed logits ``[N, V]`` with ``cu_seqlens``.
On B200 (``csrc/ctc.cu``): one CTA per sequence computes the per-frame log-sum-exp, runs the alpha and beta recursions
in shared memory over the extended label sequence and writes ``dlogits = softmax - posterior`` in the logits dtype, so
the ``[T, V]`` log-probabilities are never materialised. Scratch memory (global): per-frame log-sum-exp and the alpha
lattice ``[T, 2S+1]`` per sequence. Otherwise ``torch.nn.functional.ctc_loss`` in fp32.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import torch
import torch.nn.functional as F
from . import _lib

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


def available() -> bool:
    """library present with the CTC entry point"""
    lib = _lib.get_lib()
    return lib is not None and hasattr(lib, "rb200_ctc_loss")


def supports(logits, targets) -> bool:
    """dtype / size limits of the kernel"""
    return logits.dtype in (torch.bfloat16, torch.float32) and targets.shape[-1] <= max_target_len() and logits.shape[-1] <= 50000


def max_target_len() -> int:
    """longest label sequence the kernels handle (the gradient kernel keeps 16 * (2S+1) floats in shared memory)"""
    return 1500


class _CtcFn(torch.autograd.Function):
    """loss and gradient come out of the same launches; backward scales the stored gradient by dloss of its sequence"""

    @staticmethod
    def forward(ctx, logits_rows, cu, row_batch, lens, targets, tgt_lens, blank, max_s):
        n, v = logits_rows.shape
        b = lens.shape[0]
        logits_rows = logits_rows.contiguous()
        targets = targets.to(torch.int32).contiguous()
        if targets.dim() == 1:
            targets = targets.unsqueeze(0)
        loss = torch.empty(b, dtype=torch.float32, device=logits_rows.device)
        need_grad = logits_rows.requires_grad
        grad = torch.empty_like(logits_rows) if need_grad else None
        s_ext = 2 * max_s + 1
        scratch = torch.empty(n * (1 + 3 * s_ext) + b, dtype=torch.float32, device=logits_rows.device)
        fn = _lib.bind("rb200_ctc_loss", [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i64, _vp])
        _lib.check(fn(logits_rows.data_ptr(), 1 if logits_rows.dtype == torch.bfloat16 else 0, cu.data_ptr(), row_batch.data_ptr(),
                      targets.data_ptr(), tgt_lens.data_ptr(), loss.data_ptr(), grad.data_ptr() if grad is not None else None,
                      scratch.data_ptr(), b, n, v, targets.shape[1], max_s, blank, scratch.numel(), _lib.stream_ptr()), "ctc_loss")
        _lib.count_launch(3 if need_grad else 2)
        if need_grad:
            ctx.save_for_backward(grad, row_batch)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        grad, row_batch = ctx.saved_tensors
        lib = _lib.get_lib()
        if grad.is_cuda and lib is not None and hasattr(lib, "rb200_ctc_scale_rows") and grad.dtype in (torch.bfloat16, torch.float32):
            dl = dloss.to(torch.float32).contiguous()
            out = torch.empty_like(grad)
            fn = _lib.bind("rb200_ctc_scale_rows", [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp])
            _lib.check(fn(grad.data_ptr(), row_batch.data_ptr(), dl.data_ptr(), out.data_ptr(), grad.shape[0], grad.shape[1],
                          1 if grad.dtype == torch.bfloat16 else 0, _lib.stream_ptr()), "ctc_scale_rows")
            _lib.count_launch()
            return out, None, None, None, None, None, None, None
        scale = dloss.to(torch.float32)[row_batch.long()].unsqueeze(-1)
        return (grad.float() * scale).to(grad.dtype), None, None, None, None, None, None, None


def ctc_loss_packed(logits_rows: torch.Tensor, pack, targets: torch.Tensor, tgt_lens_host: torch.Tensor, *, blank_index: int) -> torch.Tensor:
    """
    :param logits_rows: [N, V] unnormalised
    :param pack: PackInfo of the rows
    :param targets: [B, S] (padded, any int dtype, on the device)
    :param tgt_lens_host: [B] on the host
    :return: [B] negative log likelihood (0 for infeasible alignments)
    """
    max_s = int(tgt_lens_host.max()) if tgt_lens_host.numel() else 0
    if logits_rows.is_cuda and _lib.use_native(logits_rows) and available() and supports(logits_rows, targets):
        from ..models.packing import host_to_device

        tl = host_to_device(tgt_lens_host.to(torch.int32), logits_rows.device)
        return _CtcFn.apply(logits_rows, pack.cu, pack.row_batch, pack.lens, targets, tl, blank_index, max_s)
    padded = pack.unpack(logits_rows)  # [B, T, V]
    log_probs = F.log_softmax(padded.float(), dim=-1).transpose(0, 1)
    return F.ctc_loss(log_probs, targets.long(), pack.lens_host.long(), tgt_lens_host.long().cpu(), blank=blank_index, reduction="none", zero_infinity=True)


def ctc_loss(logits: torch.Tensor, targets: torch.Tensor, in_lens: torch.Tensor, tgt_lens: torch.Tensor, *, blank_index: int,
             logits_normalized: bool = False) -> torch.Tensor:
    """padded variant: packs the valid frames and calls the packed kernel"""
    from ..models.packing import PackInfo

    # lengths are wanted on the host (layout of the packed rows): pass host tensors where they exist, a device tensor costs a
    # synchronising read here
    pack = PackInfo(in_lens.cpu(), logits.device, padded_len=logits.shape[1])
    rows = pack.pack(logits)
    return ctc_loss_packed(rows, pack, targets, tgt_lens.cpu(), blank_index=blank_index)
