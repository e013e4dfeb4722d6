"""
Attention: scaled dot-product attention, self / causal / cross / relative-positional variants, positional encodings.

Execution: the RF-level functions here work on padded named-dim tensors. ``dot_attention`` and
``RelPosSelfAttention`` hand the ``[B, H, T, D]`` blocks to :mod:`returnn_b200.ops.attention`, which on B200 runs the
fused sm_100a kernels (scores, length masks, softmax, dropout and PV in one pass; the relative-position term is
taken from a band of ``(q+v) P^T`` computed in the kernel, never materialising ``[B,H,T,2T-1]``), and otherwise a
reference implementation in torch.

Parameter layout (checkpoint compatible): ``qkv.weight [in, H*(2*Dk+Dv)]`` with the output features grouped per head as
``(q, k, v)``; ``linear_pos.weight [in, K]`` without bias; ``pos_bias_u/v [H, Dk]``.

Parity: returnn/frontend/attention.py (dot_attention :31, SelfAttention :274, CausalSelfAttention :289, RotaryPos* :414,
RelPosSelfAttention :560, CrossAttention :894, LearnedRelativePositionalEncoding :1022,
relative_positional_encoding :1146, sinusoidal_positional_encoding :1207); generic math
returnn/frontend/_backend.py:1575-1717.
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple, Union
import math
import torch
from ..tensor import Tensor, Dim, single_step_dim, batch_dim
from .module import Module
from .parameter import Parameter
from .linear import Linear
from .state import State
from . import init as _init
from ._utils import wrap, axis_of
from . import array_ as _a
from . import math_ as _m
from .dropout import dropout
from .matmul import matmul

__all__ = ["dot_attention", "SelfAttentionBase", "SelfAttention", "CausalSelfAttention", "CausalSelfAttentionState",
           "RotaryPosSelfAttention", "RotaryPosCausalSelfAttention", "RelPosSelfAttention", "RelPosCausalSelfAttention",
           "CrossAttention", "LearnedRelativePositionalEncoding", "relative_positional_encoding",
           "sinusoidal_positional_encoding", "sinusoidal_encoding"]


def _att_dropout_broadcast_default() -> bool:
    from ..config import get_global_config
    from ..utils.basic import BehaviorVersion

    cfg = get_global_config(raise_exception=False)
    if cfg and cfg.has("rf_att_dropout_broadcast"):
        return cfg.bool("rf_att_dropout_broadcast", True)
    return BehaviorVersion.get() <= 18


def _train_dropout(p: float) -> float:
    from .run_ctx import get_run_ctx

    if not p:
        return 0.0
    flag = get_run_ctx().is_train_flag_enabled(func=dropout)
    flag = bool(flag.raw_tensor) if isinstance(flag, Tensor) else bool(flag)
    return float(p) if flag else 0.0


def dot_attention(query: Tensor, keys: Tensor, values: Tensor, *, key_dim: Dim, axis: Dim, att_dropout: float = 0.0,
                  att_dropout_broadcast: Optional[bool] = None, causal_query_spatial_dim: Optional[Dim] = None,
                  scale: Optional[float] = None) -> Tensor:
    """
    softmax(query . keys * scale) . values over ``axis``.

    :param query: {..., key_dim}; dims shared with keys/values are batch dims
    :param keys: {..., axis, key_dim}
    :param values: {..., axis, v_feat}
    :param causal_query_spatial_dim: query position i only sees key positions <= i
    :return: values without axis, plus the extra query dims
    """
    if att_dropout_broadcast is None:
        att_dropout_broadcast = _att_dropout_broadcast_default()
    if scale is None:
        scale = key_dim.dimension ** -0.5
    if causal_query_spatial_dim is None and axis in query.dims:
        kv_dim = Dim(None, name="%s:kv" % axis.name)
        keys, _ = _replace(keys, axis, kv_dim)
        values, _ = _replace(values, axis, kv_dim)
        axis = kv_dim
    elif causal_query_spatial_dim is not None and causal_query_spatial_dim == axis:
        kv_dim = Dim(None, name="%s:kv" % axis.name)
        keys, _ = _replace(keys, axis, kv_dim)
        values, _ = _replace(values, axis, kv_dim)
        axis = kv_dim
    v_feat = [d for d in values.dims if d not in keys.dims]
    if not v_feat and key_dim in values.dims:
        v_feat = [key_dim]  # value and key features are the same dim (equal per-head sizes derived from one model dim)
    common = [d for d in keys.dims if d in query.dims and d not in (key_dim,)]
    q_only = [d for d in query.dims if d not in keys.dims]
    # fast path for the [batch.., T_q, D] x [batch.., T_kv, D] layout
    if len(q_only) <= 1 and len(v_feat) == 1 and not (att_dropout_broadcast and _train_dropout(att_dropout)):
        from ..ops import attention as _att

        q_sp = q_only[0] if q_only else None
        qr = query.copy_compatible_to_dims_raw(common + ([q_sp] if q_sp else []) + [key_dim])
        kr = keys.copy_compatible_to_dims_raw(common + [axis, key_dim])
        vr = values.copy_compatible_to_dims_raw(common + [axis, v_feat[0]])
        cshape = [max(a, b) for a, b in zip(qr.shape[: len(common)], kr.shape[: len(common)])]
        if not q_sp:
            qr = qr.unsqueeze(-2)
        kv_lens = _lens_for(axis, common, cshape, kr.device)
        out = _att.sdpa(qr.expand(*cshape, *qr.shape[len(common):]), kr.expand(*cshape, *kr.shape[len(common):]),
                        vr.expand(*cshape, *vr.shape[len(common):]), kv_lens=kv_lens, scale=scale,
                        causal=causal_query_spatial_dim is not None,
                        dropout_p=_train_dropout(att_dropout))
        if not q_sp:
            out = out.squeeze(-2)
        return wrap(out, common + ([q_sp] if q_sp else []) + [v_feat[0]], feature_dim=v_feat[0])
    # generic path (also: dropout mask broadcast over all but the kv axis, which has no fused form)
    energy = matmul(query, keys, reduce=key_dim) * scale
    if causal_query_spatial_dim is not None:
        from .dims import range_over_dim

        qpos = range_over_dim(causal_query_spatial_dim, device=energy.device)
        kpos = range_over_dim(axis, device=energy.device)
        energy = _a.where(_m.compare(kpos, "<=", qpos), energy, float("-inf"))
    att_weights = _m.softmax(energy, axis=axis)
    att_weights = dropout(att_weights, att_dropout, axis=att_dropout_broadcast and axis)
    att = matmul(att_weights, values, reduce=axis, use_mask=False)
    if v_feat and v_feat[0] in att.dims:
        att.feature_dim = v_feat[0]
    return att


def _replace(x: Tensor, in_dim: Dim, out_dim: Dim):
    from .dims import replace_dim

    return replace_dim(x, in_dim=in_dim, out_dim=out_dim)


def _lens_for(axis: Dim, common: Sequence[Dim], cshape, device) -> Optional[torch.Tensor]:
    """kv lengths broadcast to the batch dims, or None when unmasked"""
    if not (axis.is_dynamic() and axis.dyn_size_ext is not None and axis.dyn_size_ext.dims):
        return None
    sizes = axis.get_size_tensor(device=device)
    if not all(d in common for d in sizes.dims):
        return None
    raw = sizes.copy_compatible_to_dims_raw(list(common))
    return raw.expand(*cshape).to(torch.int32)


class SelfAttentionBase(Module):
    """shared part of the self-attention variants: qkv projection, heads, output projection"""

    def __init__(self, in_dim: Dim, proj_dim: Optional[Dim], *, key_dim_total: Dim, value_dim_total: Dim,
                 num_heads: Union[int, Dim], with_bias: bool = True, att_dropout: float = 0.1,
                 att_dropout_broadcast: Optional[bool] = None):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = proj_dim if proj_dim else value_dim_total
        if isinstance(num_heads, int):
            num_heads = Dim(num_heads, name="num_heads")
        self.key_dim_total = key_dim_total
        self.key_dim_per_head = key_dim_total.div_left(num_heads)
        self.value_dim_total = value_dim_total
        self.value_dim_per_head = value_dim_total.div_left(num_heads)
        self.num_heads = num_heads
        self.qkv_dim_total = 2 * key_dim_total + value_dim_total
        self.qkv_dim_per_head = 2 * self.key_dim_per_head + self.value_dim_per_head
        self.qkv = Linear(in_dim, self.qkv_dim_total, with_bias=with_bias)
        self.proj = Linear(value_dim_total, proj_dim, with_bias=with_bias) if proj_dim else None
        self.att_dropout = att_dropout
        if att_dropout_broadcast is None:
            att_dropout_broadcast = _att_dropout_broadcast_default()
        self.att_dropout_broadcast = att_dropout_broadcast

    def forward_qkv(self, source: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        """:return: q, k, v each {..., heads, per-head dim}"""
        qkv = self.qkv(source)
        qkv = _a.split_dims(qkv, axis=self.qkv_dim_total, dims=(self.num_heads, self.qkv_dim_per_head))
        q, k, v = _a.split(qkv, axis=self.qkv_dim_per_head,
                           out_dims=(self.key_dim_per_head, self.key_dim_per_head, self.value_dim_per_head))
        return q, k, v

    def attention(self, q: Tensor, k: Tensor, v: Tensor, *, kv_axis: Dim, causal_query_spatial_dim: Optional[Dim] = None) -> Tensor:
        """attention + merge heads + output projection"""
        att = dot_attention(q, k, v, key_dim=self.key_dim_per_head, axis=kv_axis, att_dropout=self.att_dropout,
                            att_dropout_broadcast=self.att_dropout_broadcast, causal_query_spatial_dim=causal_query_spatial_dim)
        output, _ = _a.merge_dims(att, dims=(self.num_heads, self.value_dim_per_head), out_dim=self.value_dim_total)
        if self.proj:
            output = self.proj(output)
        return output


class SelfAttention(SelfAttentionBase):
    """bidirectional self-attention over ``axis``"""

    def __call__(self, source: Tensor, *, axis: Dim) -> Tensor:
        if axis not in source.dims:
            from . import packed_mode

            pdim = packed_mode.packed_dim_of(source, axis)
            if pdim is not None:  # packed rows: attention inside every sequence, on the padded form
                return packed_mode.apply_padded(lambda padded: self(padded, axis=axis), source, pdim)
        q, k, v = self.forward_qkv(source)
        kv_axis = Dim(None, name="%s-kv" % axis.name)
        k, _ = _replace(k, axis, kv_axis)
        v, _ = _replace(v, axis, kv_axis)
        return self.attention(q, k, v, kv_axis=kv_axis)


class CausalSelfAttentionState(State):
    """accumulated keys/values and their growing axis"""

    def __init__(self, *_args, k_accum: Tensor = None, v_accum: Tensor = None, accum_axis: Dim = None):
        super().__init__(*_args)
        if not _args:
            self.k_accum = k_accum
            self.v_accum = v_accum
            self.accum_axis = accum_axis


class CausalSelfAttention(SelfAttentionBase):
    """
    Causal self-attention. ``axis`` is a whole sequence (training) or ``single_step_dim`` (incremental decoding, using
    and extending the key/value history in ``state``).
    """

    def __call__(self, source: Tensor, *, axis: Dim, state: Optional[CausalSelfAttentionState] = None) -> Tuple[Tensor, CausalSelfAttentionState]:
        q, k, v = self.forward_qkv(source)
        k, v, hist_dim, new_state, causal_dim = _causal_self_att_step(k, v, axis=axis, state=state, self=self)
        output = self.attention(q, k, v, kv_axis=hist_dim, causal_query_spatial_dim=causal_dim)
        return output, new_state

    def default_initial_state(self, *, batch_dims: Sequence[Dim]) -> CausalSelfAttentionState:
        """empty history"""
        from .const import zeros

        expand_dim = Dim(0, name="self_att_expand_dim_init")
        return CausalSelfAttentionState(
            k_accum=zeros(list(batch_dims) + [expand_dim, self.num_heads, self.key_dim_per_head]),
            v_accum=zeros(list(batch_dims) + [expand_dim, self.num_heads, self.value_dim_per_head]),
            accum_axis=expand_dim)


def _causal_self_att_step(k: Tensor, v: Tensor, *, axis: Dim, state: Optional[CausalSelfAttentionState], self):
    new_state = CausalSelfAttentionState()
    causal_dim = None
    if axis == single_step_dim:
        assert state, "%s: need state for single step" % self
        if state.accum_axis.dimension == 0:
            # first step: history is just this frame
            hist_dim = Dim(None, name="self-att-hist")
            hist_dim.dyn_size_ext = Tensor("hist:size", dims=[], dtype="int32", raw_tensor=torch.tensor(1, dtype=torch.int32))
            k = _expand_at(k, hist_dim, state.k_accum, state.accum_axis)
            v = _expand_at(v, hist_dim, state.v_accum, state.accum_axis)
        else:
            k, hist_dim = _a.cum_concat_step(k, prev_accum=state.k_accum, axis=state.accum_axis,
                                             out_spatial_dim=Dim(None, name="self-att-hist"))
            v, _ = _a.cum_concat_step(v, prev_accum=state.v_accum, axis=state.accum_axis, out_spatial_dim=hist_dim)
        new_state.k_accum, new_state.v_accum, new_state.accum_axis = k, v, hist_dim
    elif state and state.accum_axis.dimension != 0:
        raise NotImplementedError("%s: chunk-wise continuation of a non-empty history" % self)
    else:
        new_state.k_accum, new_state.v_accum, new_state.accum_axis = k, v, axis
        hist_dim = Dim(None, name="%s:kv" % axis.name)
        k, _ = _replace(k, axis, hist_dim)
        v, _ = _replace(v, axis, hist_dim)
        causal_dim = axis
    return k, v, hist_dim, new_state, causal_dim


def _expand_at(x: Tensor, new_dim: Dim, like_accum: Tensor, accum_axis: Dim) -> Tensor:
    ax = like_accum.dims.index(accum_axis)
    dims = [d for d in like_accum.dims if d != accum_axis]
    raw = x.copy_compatible_to_dims_raw(dims).unsqueeze(ax)
    dims.insert(ax, new_dim)
    return wrap(raw, dims, like=x)


def _apply_rope(x: Tensor, pos_enc: Tensor, feat_dim: Dim) -> Tensor:
    """
    Rotary position embedding: the features are D/2 complex numbers stored interleaved, ``(x[2i], x[2i+1]) = (re, im)``, and
    number i is multiplied by ``cos_i + j sin_i``, where ``pos_enc = [sin_0..sin_{D/2-1} | cos_0..cos_{D/2-1}]``
    (the layout of returnn/frontend/attention.py:535; HuggingFace's Llama stores (x[i], x[i + D/2]) instead, which is why
    its q/k projection columns are permuted on import).
    """
    half = feat_dim.div_left(2)
    sin, cos = _a.split(pos_enc, axis=feat_dim, out_dims=[half, half])
    pair = Dim(2, name="complex")
    xs = _a.split_dims(x, axis=feat_dim, dims=(half, pair))
    re, im = _a.unstack(xs, axis=pair)
    out, _ = _a.stack((re * cos - im * sin, re * sin + im * cos), out_dim=pair)
    out, _ = _a.merge_dims(out, dims=(half, pair), out_dim=feat_dim)
    return out


def _rope_base(head_dim: Dim) -> float:
    """
    ``sinusoidal_positional_encoding`` spaces its D/2 frequencies as ``base ** (-i / (D/2 - 1))``; RoPE as commonly defined
    uses ``10000 ** (-2i / D)``. Both agree for ``base = 10000 ** (1 - 2 / D)`` (returnn/frontend/attention.py:492).
    """
    return 10_000 ** (1 - 2 / head_dim.dimension)


class RotaryPosSelfAttention(SelfAttention):
    """self-attention with rotary position embedding (RoPE) on q and k"""

    def __call__(self, source: Tensor, *, axis: Dim) -> Tensor:
        q, k, v = self.forward_qkv(source)
        pos_enc = sinusoidal_positional_encoding(spatial_dim=axis, feat_dim=self.key_dim_per_head, base=_rope_base(self.key_dim_per_head), device=source.device)
        q = _apply_rope(q, pos_enc, self.key_dim_per_head)
        k = _apply_rope(k, pos_enc, self.key_dim_per_head)
        kv_axis = Dim(None, name="%s-kv" % axis.name)
        k, _ = _replace(k, axis, kv_axis)
        v, _ = _replace(v, axis, kv_axis)
        return self.attention(q, k, v, kv_axis=kv_axis)


class RotaryPosCausalSelfAttention(CausalSelfAttention):
    """causal self-attention with RoPE"""

    def __call__(self, source: Tensor, *, axis: Dim, state: Optional[CausalSelfAttentionState] = None):
        q, k, v = self.forward_qkv(source)
        if axis == single_step_dim:
            assert state
            offset = state.accum_axis.get_dim_value() if state.accum_axis.dimension != 0 else 0
            pos_enc = sinusoidal_positional_encoding(spatial_dim=single_step_dim, offset=offset, feat_dim=self.key_dim_per_head,
                                                     base=_rope_base(self.key_dim_per_head), device=source.device)
        else:
            pos_enc = sinusoidal_positional_encoding(spatial_dim=axis, feat_dim=self.key_dim_per_head, base=_rope_base(self.key_dim_per_head), device=source.device)
        q = _apply_rope(q, pos_enc, self.key_dim_per_head)
        k = _apply_rope(k, pos_enc, self.key_dim_per_head)
        k, v, hist_dim, new_state, causal_dim = _causal_self_att_step(k, v, axis=axis, state=state, self=self)
        output = self.attention(q, k, v, kv_axis=hist_dim, causal_query_spatial_dim=causal_dim)
        return output, new_state


class RelPosSelfAttention(SelfAttentionBase):
    """
    Self-attention with Transformer-XL style relative positional encoding (as in ESPnet Conformer):
    ``score[q,k] = ((q+u).k + (q+v).P[k-q]) / sqrt(Dk)``.
    """

    def __init__(self, in_dim: Dim, proj_dim: Optional[Dim], *, key_dim_total: Dim, value_dim_total: Dim,
                 num_heads: Union[int, Dim], with_bias: bool = True, with_linear_pos: bool = True,
                 with_pos_bias: bool = True, learnable_pos_emb: bool = False, learnable_pos_emb_clipping: int = 16,
                 separate_pos_emb_per_head: bool = True, pos_emb_dropout: float = 0.0, att_dropout: float = 0.1,
                 att_dropout_broadcast: Optional[bool] = None):
        super().__init__(in_dim=in_dim, proj_dim=proj_dim, key_dim_total=key_dim_total, value_dim_total=value_dim_total,
                         num_heads=num_heads, with_bias=with_bias, att_dropout=att_dropout,
                         att_dropout_broadcast=att_dropout_broadcast)
        self.separate_pos_emb_per_head = separate_pos_emb_per_head
        if with_linear_pos:
            self.pos_emb_feat_dim = self.in_dim
        elif separate_pos_emb_per_head:
            self.pos_emb_feat_dim = self.key_dim_total
        else:
            self.pos_emb_feat_dim = self.key_dim_per_head
        self.linear_pos = None
        if with_linear_pos:
            self.linear_pos = Linear(self.in_dim, self.key_dim_total if separate_pos_emb_per_head else self.key_dim_per_head, with_bias=False)
        self.learned_pos_emb = None
        if learnable_pos_emb:
            self.learned_pos_emb = LearnedRelativePositionalEncoding(self.pos_emb_feat_dim, clipping=learnable_pos_emb_clipping)
        self.pos_bias_u = None
        self.pos_bias_v = None
        if with_pos_bias:
            self.pos_bias_u = Parameter((self.num_heads, self.key_dim_per_head))
            self.pos_bias_v = Parameter((self.num_heads, self.key_dim_per_head))
            self.pos_bias_u.initial = _init.Glorot()
            self.pos_bias_v.initial = _init.Glorot()
        self.pos_emb_dropout = pos_emb_dropout

    def _pos_emb(self, axis: Dim, device) -> Tuple[Tensor, Dim]:
        if self.learned_pos_emb is not None:
            pos_emb, pos_dim = self.learned_pos_emb(query_spatial_dim=axis, key_value_spatial_dim=axis)
        else:
            pos_emb, pos_dim = relative_positional_encoding(query_spatial_dim=axis, key_value_spatial_dim=axis,
                                                            feat_dim=self.pos_emb_feat_dim, device=device)
        if self.pos_emb_dropout:
            pos_emb = dropout(pos_emb, self.pos_emb_dropout)
        if self.linear_pos is not None:
            if pos_emb.dtype != self.linear_pos.weight.dtype and not torch.is_autocast_enabled():
                pos_emb = _a.cast(pos_emb, self.linear_pos.weight.dtype)
            pos_emb = self.linear_pos(pos_emb)
        if self.separate_pos_emb_per_head:
            pos_emb = _a.split_dims(pos_emb, axis=self.key_dim_total, dims=(self.num_heads, self.key_dim_per_head))
        return pos_emb, pos_dim

    def __call__(self, source: Tensor, *, axis: Dim, **_kwargs) -> Tensor:
        if axis not in source.dims:
            from . import packed_mode

            pdim = packed_mode.packed_dim_of(source, axis)
            if pdim is not None:
                return self._call_packed(source, axis=axis, pdim=pdim)
        pos_emb, pos_dim = self._pos_emb(axis, source.device)
        q, k, v = self.forward_qkv(source)
        batch_dims = [d for d in q.dims if d not in (axis, self.num_heads, self.key_dim_per_head)]
        from ..ops import attention as _att

        H = self.num_heads
        qr = q.copy_compatible_to_dims_raw(batch_dims + [H, axis, self.key_dim_per_head])
        kr = k.copy_compatible_to_dims_raw(batch_dims + [H, axis, self.key_dim_per_head])
        vr = v.copy_compatible_to_dims_raw(batch_dims + [H, axis, self.value_dim_per_head])
        if self.separate_pos_emb_per_head:
            pr = pos_emb.copy_compatible_to_dims_raw([H, pos_dim, self.key_dim_per_head])
        else:
            pr = pos_emb.copy_compatible_to_dims_raw([pos_dim, self.key_dim_per_head]).unsqueeze(0).expand(H.dimension, -1, -1)
        bshape = list(qr.shape[: len(batch_dims)])
        lens = _lens_for(axis, batch_dims, bshape, qr.device)
        u = self.pos_bias_u.raw_tensor if self.pos_bias_u is not None else None
        vb = self.pos_bias_v.raw_tensor if self.pos_bias_v is not None else None
        p_drop = _train_dropout(self.att_dropout)
        if p_drop and self.att_dropout_broadcast:
            out = _rel_pos_att_generic(q, k, v, pos_emb, self, axis, pos_dim)
        else:
            out_raw = _att.rel_pos_attention(qr.reshape(-1, *qr.shape[len(batch_dims):]), kr.reshape(-1, *kr.shape[len(batch_dims):]),
                                             vr.reshape(-1, *vr.shape[len(batch_dims):]), pr, u, vb,
                                             lens.reshape(-1) if lens is not None else None,
                                             scale=self.key_dim_per_head.dimension ** -0.5, dropout_p=p_drop)
            out_raw = out_raw.reshape(bshape + list(out_raw.shape[1:]))
            out = wrap(out_raw, batch_dims + [H, axis, self.value_dim_per_head], feature_dim=self.value_dim_per_head)
        output, _ = _a.merge_dims(out, dims=(self.num_heads, self.value_dim_per_head), out_dim=self.value_dim_total)
        # time before features again
        if output.dims[-1] != self.value_dim_total:
            output = output.copy_transpose_to_dims([d for d in output.dims if d != self.value_dim_total] + [self.value_dim_total])
        if self.proj:
            output = self.proj(output)
        return output


def _rel_pos_self_att_call_packed(self: RelPosSelfAttention, source: Tensor, *, axis: Dim, pdim: Dim) -> Tensor:
    """
    ``source [rows, in]`` with the valid frames of all sequences back to back. With the standard configuration (sinusoidal positions
    through ``linear_pos``, both biases, a position table per head, no broadcast dropout) the packed qkv rows go straight to the
    varlen attention (``ops/attention_packed.py``: own kernels on the GPU); otherwise the padded form runs and the result is packed.
    """
    from . import packed_mode
    from ..ops import attention_packed as _ap

    p_drop = _train_dropout(self.att_dropout)
    standard = (self.linear_pos is not None and self.pos_bias_u is not None and self.pos_bias_v is not None and self.separate_pos_emb_per_head
                and self.learned_pos_emb is None and not (p_drop and self.att_dropout_broadcast)
                and self.key_dim_per_head == self.value_dim_per_head and len(source.dims) == 2)
    if not standard:
        return packed_mode.apply_padded(lambda padded: self(padded, axis=axis), source, pdim)
    info = pdim.packed_info
    pos_emb, pos_dim = self._pos_emb(axis, source.device)  # [2 T_max - 1, heads * dim] after linear_pos
    qkv = self.qkv(source)  # [rows, heads * (q | k | v)]
    H, D = self.num_heads.dimension, self.key_dim_per_head.dimension
    qkv_raw = qkv.copy_compatible_to_dims_raw([pdim, self.qkv_dim_total])
    # the kernels want (q | k | v) per head contiguous: [rows, H, 3, D], which is the layout of the fused projection
    pos_raw = pos_emb.copy_compatible_to_dims_raw([pos_dim, self.num_heads, self.key_dim_per_head]).reshape(-1, H * D).to(qkv_raw.dtype)
    out_raw = _ap.rel_pos_attention_packed(qkv_raw.contiguous(), pos_raw.contiguous(), self.pos_bias_u.raw_tensor, self.pos_bias_v.raw_tensor, info.pack,
                                           num_heads=H, head_dim=D, scale=D ** -0.5, dropout_p=p_drop)
    output = wrap(out_raw, [pdim, self.value_dim_total], feature_dim=self.value_dim_total)
    if self.proj:
        output = self.proj(output)
    return output


RelPosSelfAttention._call_packed = _rel_pos_self_att_call_packed


def _rel_pos_enc_shift(x: Tensor, axis: Dim, pos_emb_spatial_dim: Dim, hist_dim: Dim) -> Tensor:
    """[.., T, 2T-1] -> [.., T, T']: entry (q, k) takes column k - q + T - 1"""
    T = axis.get_dim_value()
    rest = [d for d in x.dims if d not in (axis, pos_emb_spatial_dim)]
    raw = x.copy_compatible_to_dims_raw(rest + [axis, pos_emb_spatial_dim])
    qi = torch.arange(T, device=raw.device)[:, None]
    ki = torch.arange(hist_dim.get_dim_value(), device=raw.device)[None, :]
    idx = (ki - qi + T - 1).expand(*raw.shape[:-2], -1, -1)
    return wrap(torch.gather(raw, -1, idx), rest + [axis, hist_dim])


def _rel_pos_att_generic(q, k, v, pos_emb, self: RelPosSelfAttention, axis: Dim, pos_dim: Dim) -> Tensor:
    hist_dim = Dim(None, name="%s:kv" % axis.name)
    k, _ = _replace(k, axis, hist_dim)
    v, _ = _replace(v, axis, hist_dim)
    q_u = (q + self.pos_bias_u) if self.pos_bias_u is not None else q
    q_v = (q + self.pos_bias_v) if self.pos_bias_v is not None else q
    ac = matmul(q_u, k, reduce=self.key_dim_per_head)
    bd = matmul(q_v, pos_emb, reduce=self.key_dim_per_head)
    bd = _rel_pos_enc_shift(bd, axis, pos_dim, hist_dim)
    scores = (ac + bd) * (self.key_dim_per_head.dimension ** -0.5)
    w = _m.softmax(scores, axis=hist_dim)
    w = dropout(w, self.att_dropout, axis=self.att_dropout_broadcast and hist_dim)
    att = matmul(w, v, reduce=hist_dim, use_mask=False)
    att.feature_dim = self.value_dim_per_head
    return att


class RelPosCausalSelfAttention(CausalSelfAttention):
    """causal self-attention with learned / sinusoidal relative positions (full-sequence mode)"""

    def __init__(self, in_dim: Dim, proj_dim: Optional[Dim], *, key_dim_total: Dim, value_dim_total: Dim,
                 num_heads: Union[int, Dim], with_bias: bool = True, with_linear_pos: bool = True, with_pos_bias: bool = True,
                 learnable_pos_emb: bool = False, learnable_pos_emb_clipping: int = 16, separate_pos_emb_per_head: bool = True,
                 pos_emb_dropout: float = 0.0, att_dropout: float = 0.1):
        super().__init__(in_dim=in_dim, proj_dim=proj_dim, key_dim_total=key_dim_total, value_dim_total=value_dim_total,
                         num_heads=num_heads, with_bias=with_bias, att_dropout=att_dropout)
        rel = RelPosSelfAttention.__new__(RelPosSelfAttention)
        self._rel_holder = (rel,)  # in a tuple: not a sub-module, its parameters are registered on self below
        RelPosSelfAttention.__init__(rel, in_dim, proj_dim, key_dim_total=key_dim_total, value_dim_total=value_dim_total,
                                     num_heads=self.num_heads, with_bias=with_bias, with_linear_pos=with_linear_pos,
                                     with_pos_bias=with_pos_bias, learnable_pos_emb=learnable_pos_emb,
                                     learnable_pos_emb_clipping=learnable_pos_emb_clipping,
                                     separate_pos_emb_per_head=separate_pos_emb_per_head, pos_emb_dropout=pos_emb_dropout,
                                     att_dropout=att_dropout)
        # share the projections: one set of parameters
        self.linear_pos = rel.linear_pos
        self.learned_pos_emb = rel.learned_pos_emb
        self.pos_bias_u = rel.pos_bias_u
        self.pos_bias_v = rel.pos_bias_v
        del rel.qkv, rel.proj

    def __call__(self, source: Tensor, *, axis: Dim, state: Optional[CausalSelfAttentionState] = None):
        assert axis != single_step_dim, "%s: stepwise mode is not supported" % self
        rel = self._rel_holder[0]
        rel.qkv, rel.proj = self.qkv, self.proj
        try:
            pos_emb, pos_dim = rel._pos_emb(axis, source.device)
            q, k, v = self.forward_qkv(source)
            hist_dim = Dim(None, name="%s:kv" % axis.name)
            k2, _ = _replace(k, axis, hist_dim)
            v2, _ = _replace(v, axis, hist_dim)
            q_u = (q + self.pos_bias_u) if self.pos_bias_u is not None else q
            q_v = (q + self.pos_bias_v) if self.pos_bias_v is not None else q
            ac = matmul(q_u, k2, reduce=self.key_dim_per_head)
            bd = _rel_pos_enc_shift(matmul(q_v, pos_emb, reduce=self.key_dim_per_head), axis, pos_dim, hist_dim)
            scores = (ac + bd) * (self.key_dim_per_head.dimension ** -0.5)
            from .dims import range_over_dim

            qpos = range_over_dim(axis, device=scores.device)
            kpos = range_over_dim(hist_dim, device=scores.device)
            scores = _a.where(_m.compare(kpos, "<=", qpos), scores, float("-inf"))
            w = dropout(_m.softmax(scores, axis=hist_dim), self.att_dropout, axis=self.att_dropout_broadcast and hist_dim)
            att = matmul(w, v2, reduce=hist_dim, use_mask=False)
            output, _ = _a.merge_dims(att, dims=(self.num_heads, self.value_dim_per_head), out_dim=self.value_dim_total)
            if self.proj:
                output = self.proj(output)
        finally:
            del rel.qkv, rel.proj
        new_state = CausalSelfAttentionState(k_accum=k, v_accum=v, accum_axis=axis)
        return output, new_state


class CrossAttention(Module):
    """
    Encoder-decoder attention. ``transform_encoder`` computes keys/values once per sequence;
    ``__call__`` attends from decoder queries.
    """

    def __init__(self, encoder_dim: Dim, query_in_dim: Dim, proj_dim: Optional[Dim], *, key_dim_total: Dim,
                 value_dim_total: Dim, num_heads: Union[int, Dim], with_bias: bool = True, att_dropout: float = 0.1,
                 att_dropout_broadcast: Optional[bool] = None):
        super().__init__()
        self.encoder_dim = encoder_dim
        self.query_in_dim = query_in_dim
        self.out_dim = proj_dim if proj_dim else value_dim_total
        if isinstance(num_heads, int):
            num_heads = Dim(num_heads, name="num_heads")
        self.key_dim_total = key_dim_total
        self.key_dim_per_head = key_dim_total.div_left(num_heads)
        self.value_dim_total = value_dim_total
        self.value_dim_per_head = value_dim_total.div_left(num_heads)
        self.num_heads = num_heads
        self.kv_dim_total = key_dim_total + value_dim_total
        self.kv_dim_per_head = self.key_dim_per_head + self.value_dim_per_head
        self.kv = Linear(encoder_dim, self.kv_dim_total, with_bias=with_bias)
        self.q = Linear(query_in_dim, self.key_dim_total, with_bias=with_bias)
        # the kv weight has 2x the fan-out of separate k and v projections: compensate in the scale
        self.kv.weight.initial = _init.Glorot(scale=3 / 4)
        self.q.weight.initial = _init.Glorot(scale=1 / 2)
        self.proj = Linear(value_dim_total, proj_dim, with_bias=with_bias) if proj_dim else None
        self.att_dropout = att_dropout
        if att_dropout_broadcast is None:
            att_dropout_broadcast = _att_dropout_broadcast_default()
        self.att_dropout_broadcast = att_dropout_broadcast

    def transform_encoder(self, encoder: Tensor, *, axis: Dim) -> State:
        """:return: State(k, v, kv_axis)"""
        k, v = self.forward_kv(encoder)
        return State(k=k, v=v, kv_axis=axis)

    def forward_kv(self, source: Tensor) -> Tuple[Tensor, Tensor]:
        """k, v {..., heads, per-head}"""
        kv = self.kv(source)
        kv = _a.split_dims(kv, axis=self.kv_dim_total, dims=(self.num_heads, self.kv_dim_per_head))
        k, v = _a.split(kv, axis=self.kv_dim_per_head, out_dims=(self.key_dim_per_head, self.value_dim_per_head))
        return k, v

    def forward_query(self, source: Tensor) -> Tensor:
        """q {..., heads, per-head}"""
        q = self.q(source)
        return _a.split_dims(q, axis=self.key_dim_total, dims=(self.num_heads, self.key_dim_per_head))

    def __call__(self, q: Tensor, encoder: State) -> Tensor:
        q = self.forward_query(q)
        return self.attention(q=q, **encoder)

    def attention(self, q: Tensor, k: Tensor, v: Tensor, *, kv_axis: Dim) -> Tensor:
        """attention + merge heads + projection"""
        att = dot_attention(q, k, v, key_dim=self.key_dim_per_head, axis=kv_axis, att_dropout=self.att_dropout,
                            att_dropout_broadcast=self.att_dropout_broadcast)
        output, _ = _a.merge_dims(att, dims=(self.num_heads, self.value_dim_per_head), out_dim=self.value_dim_total)
        if self.proj:
            output = self.proj(output)
        return output


class LearnedRelativePositionalEncoding(Module):
    """learned embedding per clipped relative distance"""

    def __init__(self, feat_dim: Dim, *, clipping: int = 16, dtype: Optional[str] = None, causal: bool = False):
        super().__init__()
        self.feat_dim = feat_dim
        self.clipping = clipping
        self.clipped_spatial_dim = Dim((1 if causal else 2) * clipping + 1, name="learned-rel-pos")
        self.causal = causal
        self.pos_emb = Parameter((self.clipped_spatial_dim, self.feat_dim), dtype=dtype)
        self.pos_emb.initial = _init.Glorot()

    def __call__(self, *, query_spatial_dim: Dim, key_value_spatial_dim: Dim, query_offset: Optional[int] = None) -> Tuple[Tensor, Dim]:
        """:return: [q_len + kv_len - 1, feat_dim] in the same compact layout as relative_positional_encoding"""
        indices, out_spatial_dim = _make_indices(query_spatial_dim, key_value_spatial_dim, query_offset, device=self.pos_emb.device)
        raw = indices.raw_tensor.clamp(-self.clipping, 0 if self.causal else self.clipping) + self.clipping
        enc = _a.gather(self.pos_emb, indices=wrap(raw, indices.dims, sparse_dim=self.clipped_spatial_dim), axis=self.clipped_spatial_dim)
        return enc, out_spatial_dim

    def full_matrix(self, *, query_spatial_dim: Dim, key_value_spatial_dim: Dim, query_offset: int = 0) -> Tensor:
        """:return: [q_len, kv_len, feat_dim]"""
        from .dims import range_over_dim

        kv = range_over_dim(key_value_spatial_dim, device=self.pos_emb.device)
        qv = range_over_dim(query_spatial_dim, device=self.pos_emb.device)
        idx = _m.combine(kv, "-", qv + query_offset)
        raw = idx.raw_tensor.clamp(-self.clipping, 0 if self.causal else self.clipping) + self.clipping
        return _a.gather(self.pos_emb, indices=wrap(raw, idx.dims, sparse_dim=self.clipped_spatial_dim), axis=self.clipped_spatial_dim)


def _make_indices(query_spatial_dim: Dim, key_value_spatial_dim: Dim, query_offset=None, device=None) -> Tuple[Tensor, Dim]:
    """relative distances k - q for the compact [q_len + kv_len - 1] layout"""
    if query_spatial_dim == single_step_dim:
        n = key_value_spatial_dim.get_dim_value()
        raw = torch.arange(n, device=device, dtype=torch.int32) - (n - 1)
        return wrap(raw, [key_value_spatial_dim]), key_value_spatial_dim
    qn = query_spatial_dim.get_dim_value()
    kn = key_value_spatial_dim.get_dim_value()
    out_dim = Dim(None, name="2*%s-1" % query_spatial_dim.name if query_spatial_dim == key_value_spatial_dim else "%s+%s-1" % (query_spatial_dim.name, key_value_spatial_dim.name))
    out_dim.dyn_size_ext = Tensor("relpos:size", dims=[], dtype="int32", raw_tensor=torch.tensor(qn + kn - 1, dtype=torch.int32))
    raw = torch.arange(-(qn - 1), kn, device=device, dtype=torch.int32)
    if query_offset:
        raw = raw - query_offset
    return wrap(raw, [out_dim]), out_dim


_rel_pos_cache = {}


def relative_positional_encoding(*, query_spatial_dim: Dim, key_value_spatial_dim: Dim, feat_dim: Dim,
                                 query_offset: int = 0, dtype: Optional[str] = None, device: Optional[str] = None) -> Tuple[Tensor, Dim]:
    """
    Sinusoidal encoding of the relative distances ``k - q`` in ``[-(q_len-1), kv_len-1]``:
    first half of the features sin, second half cos, frequencies ``1e4^(-2i/F)``.

    :return: [q_len + kv_len - 1, feat_dim] and that spatial dim; distance 0 is at index q_len - 1
    """
    from ._utils import get_default_float_dtype, torch_dtype

    dtype = dtype or get_default_float_dtype()
    if query_spatial_dim == single_step_dim:
        qn, kn = 1, key_value_spatial_dim.get_dim_value()
    else:
        qn, kn = query_spatial_dim.get_dim_value(), key_value_spatial_dim.get_dim_value()
    key = (id(query_spatial_dim.get_same_base()), id(key_value_spatial_dim.get_same_base()), qn, kn, id(feat_dim.get_same_base()), query_offset, dtype, str(device))
    hit = _rel_pos_cache.get(key)
    if hit is not None:
        return hit
    indices, out_dim = _make_indices(query_spatial_dim, key_value_spatial_dim, query_offset, device=device)
    F2 = feat_dim.dimension // 2
    div_term = torch.exp(torch.arange(F2, device=device, dtype=torch.float32) * -(2.0 * math.log(1e4) / feat_dim.dimension))
    arg = indices.raw_tensor.to(torch.float32)[:, None] * div_term[None, :]
    emb = torch.cat([torch.sin(arg), torch.sin(arg + math.pi / 2.0)], dim=-1).to(torch_dtype(dtype))
    res = (wrap(emb, [out_dim, feat_dim], feature_dim=feat_dim), out_dim)
    if len(_rel_pos_cache) > 128:
        _rel_pos_cache.clear()
    _rel_pos_cache[key] = res
    return res


def sinusoidal_positional_encoding(*, spatial_dim: Dim, feat_dim: Dim, offset=None, base: Union[int, float] = 1e4,
                                   dtype: Optional[str] = None, device: Optional[str] = None) -> Tensor:
    """absolute sinusoidal encoding: [spatial_dim, feat_dim], or [feat_dim] for single_step_dim (offset = position)"""
    from .dims import range_over_dim
    from ._utils import convert_to_tensor

    if spatial_dim == single_step_dim:
        assert offset is not None
        indices = convert_to_tensor(offset, device=device) if not isinstance(offset, Tensor) else offset
        if device is not None and isinstance(indices.raw_tensor, torch.Tensor) and str(indices.raw_tensor.device).split(":")[0] != str(device).split(":")[0]:
            from ..tensor.utils import host_to_device

            indices = indices.copy_with_raw(host_to_device(indices.raw_tensor, device))
    else:
        indices = range_over_dim(spatial_dim, device=device)
        if offset is not None:
            indices = indices + offset
    return sinusoidal_encoding(indices, base=base, feat_dim=feat_dim, dtype=dtype)


def sinusoidal_encoding(indices: Tensor, *, feat_dim: Dim, base: Union[int, float] = 1e4, dtype: Optional[str] = None,
                        allow_single_step: bool = True) -> Tensor:
    """sin | cos encoding of arbitrary integer positions: dims = indices.dims + [feat_dim]"""
    from ._utils import get_default_float_dtype, torch_dtype

    dtype = dtype or get_default_float_dtype()
    F2 = feat_dim.dimension // 2
    raw = indices.raw_tensor
    # angle of unit i: position * base ** (-i / (F/2 - 1)), i.e. the last unit has the wavelength 2 pi base exactly
    # (reference: returnn/frontend/attention.py:1281-1283; not the F/2 in the denominator of the original Transformer paper)
    div_term = torch.exp(torch.arange(F2, device=raw.device, dtype=torch.float32) * -(math.log(base) / max(F2 - 1, 1)))
    arg = raw.to(torch.float32).unsqueeze(-1) * div_term
    emb = torch.cat([torch.sin(arg), torch.sin(arg + math.pi / 2.0)], dim=-1).to(torch_dtype(dtype))
    return wrap(emb, list(indices.dims) + [feat_dim], feature_dim=feat_dim)
