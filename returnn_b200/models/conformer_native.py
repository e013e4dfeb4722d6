"""
Binding of the native Conformer encoder executor (``csrc/encoder_exec.cu``).

The executor runs the whole layer stack, forward or backward, as one native call that launches a fixed kernel sequence
on the current stream; Python only allocates two buffers per pass. It needs

- the parameters in a :class:`returnn_b200.parallel.arena.ParamArena` (fp32 master weights, fp32 gradient arena into
  which the backward pass accumulates directly, bf16 shadow of the weights for the GEMM operands),
- the standard layer configuration (:func:`returnn_b200.models.conformer_fused.supports_fused`), training mode.

Everything else (other configurations, evaluation, CPU) runs the per-op path of :mod:`returnn_b200.models.conformer_fused`.
"""

from __future__ import annotations
from typing import Optional
import ctypes
import os
import numpy
import torch
from ..ops import _lib
from ..ops import gemm as _gemm
from ..ops.elementwise import _seed_tensor
from ..parallel import arena as _arena
from .packing import PackInfo

ENABLED = os.environ.get("RETURNN_B200_NATIVE_ENCODER", "1") == "1"
_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong

# parameter slots per layer, in the order of the enum in csrc/encoder_exec.cu
_SLOTS = [
    "ffn1_layer_norm.scale", "ffn1_layer_norm.bias", "ffn1.linear_ff.weight", "ffn1.linear_ff.bias", "ffn1.linear_out.weight", "ffn1.linear_out.bias",
    "self_att_layer_norm.scale", "self_att_layer_norm.bias", "self_att.qkv.weight", "self_att.qkv.bias", "self_att.linear_pos.weight",
    "self_att.pos_bias_u", "self_att.pos_bias_v", "self_att.proj.weight", "self_att.proj.bias",
    "conv_layer_norm.scale", "conv_layer_norm.bias", "conv_block.positionwise_conv1.weight", "conv_block.positionwise_conv1.bias",
    "conv_block.depthwise_conv.filter", "conv_block.depthwise_conv.bias", "conv_block.norm.gamma", "conv_block.norm.beta",
    "conv_block.positionwise_conv2.weight", "conv_block.positionwise_conv2.bias",
    "ffn2_layer_norm.scale", "ffn2_layer_norm.bias", "ffn2.linear_ff.weight", "ffn2.linear_ff.bias", "ffn2.linear_out.weight", "ffn2.linear_out.bias",
    "final_layer_norm.scale", "final_layer_norm.bias", "conv_block.norm.running_mean", "conv_block.norm.running_variance",
]
_GEMM_WEIGHTS = {"ffn1.linear_ff.weight", "ffn1.linear_out.weight", "self_att.qkv.weight", "self_att.linear_pos.weight", "self_att.proj.weight",
                 "conv_block.positionwise_conv1.weight", "conv_block.positionwise_conv2.weight", "ffn2.linear_ff.weight", "ffn2.linear_out.weight"}


class EncDims(ctypes.Structure):
    """mirror of ``RbEncDims``"""

    _fields_ = [(n, ctypes.c_int) for n in ("n_rows", "batch", "D", "F", "H", "Dh", "conv_k", "max_len", "R", "n_layers", "training", "n_launch")] + \
               [(n, ctypes.c_float) for n in ("ln_eps", "p_res", "p_ff", "p_att", "bn_eps", "bn_momentum", "att_scale", "ff_res_scale")]


def _get_attr_path(obj, path: str):
    for part in path.split("."):
        obj = getattr(obj, part, None)
        if obj is None:
            return None
    return obj


class NativeEncoderPlan:
    """parameter address table of one encoder over one arena; rebuilt when the arena changes"""

    def __init__(self, enc, arena: "_arena.ParamArena"):
        self.arena = arena
        layers = list(enc.layers._get_modules().values())
        self.n_layers = len(layers)
        first = layers[0]
        sa = first.self_att
        self.D = enc.out_dim.dimension
        self.F = first.ffn1.linear_ff.out_dim.dimension
        self.H = sa.num_heads.dimension
        self.Dh = sa.key_dim_per_head.dimension
        self.conv_k = first.conv_block.depthwise_conv.filter_size[0].dimension
        self.ln_eps = float(first.ffn1_layer_norm.eps)
        self.p_res = float(first.dropout)
        self.p_ff = float(first.ffn1.dropout)
        self.p_att = float(sa.att_dropout)
        self.bn_eps = float(first.conv_block.norm.eps)
        self.bn_momentum = float(first.conv_block.norm.momentum)
        self.ok = True
        shadow = arena.shadow_bf16()
        base_p, base_g, base_s = arena.flat_param.data_ptr(), arena.flat_grad.data_ptr(), shadow.data_ptr()
        n_bytes = arena.flat_param.numel() * 4
        tab = numpy.zeros((self.n_layers, len(_SLOTS), 3), dtype=numpy.int64)
        for li, layer in enumerate(layers):
            if (float(layer.dropout), float(layer.ffn1.dropout), float(layer.self_att.att_dropout)) != (self.p_res, self.p_ff, self.p_att):
                self.ok = False
            for si, path in enumerate(_SLOTS):
                p = _get_attr_path(layer, path)
                if p is None:
                    continue
                raw = p.raw_tensor
                if raw.dtype != torch.float32 or not raw.is_contiguous():
                    self.ok = False
                    continue
                addr = raw.data_ptr()
                tab[li, si, 0] = addr
                off = addr - base_p
                in_arena = 0 <= off < n_bytes
                if raw.requires_grad:
                    if not in_arena:
                        self.ok = False  # a trainable parameter outside the arena has no gradient slot
                        continue
                    tab[li, si, 1] = base_g + off
                if path in _GEMM_WEIGHTS:
                    if not in_arena:
                        self.ok = False
                        continue
                    tab[li, si, 2] = base_s + off // 2
        self.table = tab
        self.key = (base_p, base_g, base_s)
        # trainable parameters per layer (for the gradient reducer's bookkeeping)
        self.layer_params = []
        for layer in layers:
            ps = []
            for path in _SLOTS:
                p = _get_attr_path(layer, path)
                if p is not None and p.raw_tensor.requires_grad:
                    ps.append(p.raw_tensor)
            self.layer_params.append(ps)

    def still_valid(self) -> bool:
        """the arena buffers are the ones the table points into"""
        a = self.arena
        return self.key == (a.flat_param.data_ptr(), a.flat_grad.data_ptr(), a.shadow_bf16().data_ptr())


def get_plan(enc) -> Optional[NativeEncoderPlan]:
    """plan for this encoder if its parameters live in an arena with fp32 gradients on a CUDA device"""
    if not ENABLED or not _gemm.ENABLED:
        return None
    layers = list(enc.layers._get_modules().values())
    if not layers:
        return None
    probe = layers[0].ffn1.linear_ff.weight.raw_tensor
    if not probe.is_cuda:
        return None
    lib = _lib.get_lib()
    if lib is None or not hasattr(lib, "rb200_enc_forward"):
        return None
    ar = _arena.find_arena(probe)
    if ar is None or ar.dtype != torch.float32 or ar.grad_dtype != torch.float32:
        return None
    plan = getattr(enc, "_native_plan", None)
    if plan is None or plan.arena is not ar or not plan.still_valid():
        plan = NativeEncoderPlan(enc, ar)
        enc._native_plan = plan
    return plan if plan.ok else None


def _bind():
    lib = _lib.get_lib(required=True)
    sizes = _lib.bind("rb200_enc_sizes", [_vp, _vp, _vp, _vp, _vp, _vp])
    fwd = _lib.bind("rb200_enc_forward", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp])
    bwd = _lib.bind("rb200_enc_backward", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp])
    return lib, sizes, fwd, bwd


class _EncoderStackFn(torch.autograd.Function):
    """layer stack as one differentiable op w.r.t. its input; parameter gradients go to the arena directly"""

    @staticmethod
    def forward(ctx, x0, sinus, plan: NativeEncoderPlan, pack: PackInfo, grad_ready_cb):
        _, f_sizes, f_fwd, _ = _bind()
        dev = x0.device
        x0 = x0.contiguous()
        sinus = sinus.contiguous()
        assert x0.dtype == torch.bfloat16 and sinus.dtype == torch.bfloat16 and x0.shape == (pack.n, plan.D)
        d = EncDims(n_rows=pack.n, batch=pack.batch, D=plan.D, F=plan.F, H=plan.H, Dh=plan.Dh, conv_k=plan.conv_k, max_len=pack.max_len,
                    R=sinus.shape[0], n_layers=plan.n_layers, training=1, n_launch=0, ln_eps=plan.ln_eps, p_res=plan.p_res, p_ff=plan.p_ff,
                    p_att=plan.p_att, bn_eps=plan.bn_eps, bn_momentum=plan.bn_momentum, att_scale=plan.Dh ** -0.5, ff_res_scale=0.5)
        out5 = (ctypes.c_longlong * 5)()
        addr = ctypes.addressof(out5)
        _lib.check(f_sizes(ctypes.addressof(d), addr, addr + 8, addr + 16, addr + 24, addr + 32), "enc_sizes")
        saved_bytes, tmp_fwd, tmp_bwd, out_off, rng_count = [int(v) for v in out5]
        plan.arena.sync_shadow()
        saved = torch.empty(saved_bytes, dtype=torch.uint8, device=dev)
        tmp = torch.empty(tmp_fwd, dtype=torch.uint8, device=dev)
        seed = _seed_tensor(dev)
        off = seed[1:2].clone()
        seed[1] += rng_count
        st = _gemm.status_tensor(dev)
        n_launch = ctypes.c_int(0)
        tab = plan.table
        _lib.check(f_fwd(ctypes.addressof(d), tab.ctypes.data, x0.data_ptr(), sinus.data_ptr(), pack.lens.data_ptr(), pack.row_batch.data_ptr(),
                         pack.row_pos.data_ptr(), saved.data_ptr(), tmp.data_ptr(), seed.data_ptr(), off.data_ptr(), st.data_ptr(),
                         ctypes.addressof(n_launch), _lib.stream_ptr()), "enc_forward")
        _lib.count_launch(n_launch.value)
        out = saved[out_off: out_off + pack.n * plan.D * 2].view(torch.bfloat16).view(pack.n, plan.D)
        ctx.plan, ctx.pack, ctx.dims, ctx.tmp_bwd, ctx.cb = plan, pack, d, tmp_bwd, grad_ready_cb
        ctx.save_for_backward(x0, sinus, saved, off)
        return out

    @staticmethod
    def backward(ctx, d_out):
        _, _, _, f_bwd = _bind()
        x0, sinus, saved, off = ctx.saved_tensors
        plan, pack, d = ctx.plan, ctx.pack, ctx.dims
        dev = d_out.device
        dx = d_out.to(torch.bfloat16).contiguous().clone()
        tmp = torch.empty(ctx.tmp_bwd, dtype=torch.uint8, device=dev)
        seed = _seed_tensor(dev)
        st = _gemm.status_tensor(dev)
        n_launch = ctypes.c_int(0)
        tab = plan.table
        # with a gradient-ready callback (bucketed all-reduce) the stack is walked in chunks, else in one call
        step = 1 if ctx.cb is not None else plan.n_layers
        hi = plan.n_layers
        while hi > 0:
            lo = max(0, hi - step)
            _lib.check(f_bwd(ctypes.addressof(d), tab.ctypes.data, x0.data_ptr(), sinus.data_ptr(), pack.lens.data_ptr(),
                             pack.row_batch.data_ptr(), pack.row_pos.data_ptr(), saved.data_ptr(), tmp.data_ptr(), dx.data_ptr(), lo, hi,
                             seed.data_ptr(), off.data_ptr(), st.data_ptr(), ctypes.addressof(n_launch), _lib.stream_ptr()), "enc_backward")
            _lib.count_launch(n_launch.value)
            if ctx.cb is not None:
                ctx.cb(lo, hi)
            hi = lo
        return dx, None, None, None, None


def encoder_stack(x0: torch.Tensor, sinus: torch.Tensor, plan: NativeEncoderPlan, pack: PackInfo, grad_ready_cb=None) -> torch.Tensor:
    """
    :param x0: [N, D] bf16 packed rows entering the first layer
    :param sinus: [2*L-1, D] bf16 sinusoidal relative position table, L >= pack.max_len
    :param grad_ready_cb: ``cb(layer_lo, layer_hi)`` called during backward once the parameter gradients of these layers are complete
    :return: [N, D] bf16 output of the last layer
    """
    if grad_ready_cb is None:
        from ..parallel import grad_reducer as _gr

        if _gr.get_active() is not None:
            def grad_ready_cb(lo, hi):
                for li in range(lo, hi):
                    _gr.notify_grads_written(plan.layer_params[li])
    return _EncoderStackFn.apply(x0, sinus, plan, pack, grad_ready_cb)


def profile_ops(enable: bool):
    """
    Per-op timing of the executor calls (events between the ops of every forward/backward call; each call then ends with a
    stream synchronisation, so leave it off for throughput measurements). Enabling clears the table.
    """
    import ctypes
    from ..ops import _lib

    fn = _lib.bind("rb200_enc_profile_enable", [ctypes.c_int])
    _lib.check(fn(1 if enable else 0), "enc_profile_enable")


def profile_report() -> dict:
    """:return: ``{op tag: (calls, device milliseconds, host milliseconds spent issuing)}`` collected since :func:`profile_ops` was enabled"""
    import ctypes
    from ..ops import _lib

    fn = _lib.bind("rb200_enc_profile_report", [ctypes.c_char_p, ctypes.c_int])
    size = fn(None, 0)
    buf = ctypes.create_string_buffer(size + 16)
    fn(buf, size + 16)
    res = {}
    for line in buf.value.decode("utf8").splitlines():
        tag, count, ms, host = line.rsplit(" ", 3)
        res[tag] = (int(count), float(ms), float(host))
    return res
