"""
Label-synchronous beam search with ONE CUDA-graph replay per output label.

Decoding with the RF step interface issues a few hundred small kernels per label from Python, grows the key/value caches by
concatenation and asks the device twice per label whether to stop; a label then costs milliseconds of host time while the
device idles. Here the decoder step is restated over static buffers, so that the whole label step (embedding, all layers,
output layer, log-softmax + top-k over beam x vocabulary, reordering of the caches by the back-pointers, bookkeeping of
scores / lengths / history) is one fixed sequence of kernels on fixed addresses. It is captured once and replayed per label;
the host looks at the ``finished`` flags only every few labels.

* :class:`StaticTransformerDecoderStep` takes its weights from an RF :class:`TransformerDecoder` (the standard layer: causal
  self-attention, cross-attention, feed-forward, layer norms, sinusoidal or no absolute positions). Self-attention keys / values live
  in preallocated ``[layers, hyps, heads, max_steps, dim]`` caches written at the device-side step counter; attention runs over the
  full ``max_steps`` with a mask ``position <= step``. Cross-attention keys / values are computed once from the encoder output.
* :func:`beam_search_static` runs the search on such a step object; ``use_graph=None`` captures on CUDA and runs the same code
  eagerly on the CPU (where it is the test oracle against the RF decoder).

Reference for what is computed: returnn/frontend/decoder/transformer.py:216-258 (decoder step), demos/demo-rf-pt-benchmark.py:410-474
(the search loop), returnn/torch/util/graph_capture.py (static buffers + replay, there for the train step).
"""

from __future__ import annotations
from typing import List, Optional, Tuple
import math
import torch
import torch.nn.functional as F

from ..ops import seq_ops, _lib

__all__ = ["StaticTransformerDecoderStep", "beam_search_static"]


def _lin(mod):
    """(weight [in, out], bias or None) of an rf.Linear as raw tensors"""
    w = mod.weight.raw_tensor
    if tuple(mod.weight.dims) != (mod.in_dim, mod.out_dim):  # shared with an embedding: stored [out, in]
        w = w.t()
    return w, (mod.bias.raw_tensor if mod.with_bias else None)


def _norm(mod):
    """(kind, scale, bias, eps) of LayerNorm / RMSNorm"""
    name = type(mod).__name__
    if name == "LayerNorm":
        return "ln", mod.scale.raw_tensor, mod.bias.raw_tensor if getattr(mod, "bias", None) is not None else None, mod.eps
    if name == "RMSNorm":
        return "rms", mod.scale.raw_tensor, None, mod.eps
    raise TypeError("static decoder step: unsupported norm %r" % (mod,))


def _apply_norm(x, spec):
    kind, scale, bias, eps = spec
    if kind == "ln":
        return F.layer_norm(x, (x.shape[-1],), scale.to(x.dtype), bias.to(x.dtype) if bias is not None else None, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * scale.to(x.dtype)


def _activation(fn):
    name = getattr(fn, "__name__", type(fn).__name__).lower()
    table = {"relu": F.relu, "gelu": F.gelu, "swish": F.silu, "silu": F.silu, "tanh": torch.tanh, "identity": lambda x: x}
    if name not in table:
        raise TypeError("static decoder step: unsupported feed-forward activation %r" % (fn,))
    return table[name]


class StaticTransformerDecoderStep:
    """see the module docstring"""

    def __init__(self, decoder, *, enc: Optional[torch.Tensor], enc_lens: Optional[torch.Tensor], num_hyps: int, max_steps: int,
                 dtype: Optional[torch.dtype] = None):
        """
        :param decoder: rf TransformerDecoder
        :param enc: [num_seqs, T_enc, enc_dim] encoder output with ``num_hyps % num_seqs == 0``: hypotheses
            ``i * group .. (i + 1) * group`` (``group = num_hyps // num_seqs``, the beam size) belong to sequence ``i`` and share its
            cross-attention keys / values, which are stored once per sequence. (None: decoder without cross-attention)
        :param enc_lens: [num_seqs] valid encoder frames
        :param max_steps: capacity of the self-attention caches = longest output
        """
        from ..frontend.attention import CausalSelfAttention, RotaryPosCausalSelfAttention, RelPosCausalSelfAttention
        from ..frontend.decoder.transformer import FeedForward

        self.N, self.L = num_hyps, max_steps
        self.num_seqs = enc.shape[0] if enc is not None else num_hyps
        assert num_hyps % self.num_seqs == 0, "num_hyps %i is not a multiple of the number of sequences %i" % (num_hyps, self.num_seqs)
        self.group = num_hyps // self.num_seqs
        emb = decoder.input_embedding.weight.raw_tensor
        self.device = emb.device
        self.dtype = dtype or emb.dtype
        cast = lambda t: None if t is None else t.detach().to(self.dtype)  # noqa: E731
        if decoder.input_embedding_proj is not None:
            raise TypeError("static decoder step: embed_dim != model_dim is not covered")
        self.emb = cast(emb)
        self.emb_scale = float(decoder.input_embedding_scale)
        self.D = self.emb.shape[1]
        self.vocab = decoder.vocab_dim.dimension
        if decoder.pos_enc is None:
            self.pos_table = None
        else:
            from ..frontend.attention import sinusoidal_positional_encoding
            from ..tensor import Dim

            fn = decoder.pos_enc
            base_fn = getattr(fn, "func", fn)
            if base_fn is not sinusoidal_positional_encoding:
                raise TypeError("static decoder step: positional encoding %r is not covered" % (fn,))
            steps = Dim(max_steps, name="steps")
            self.pos_table = cast(fn(spatial_dim=steps, device=str(self.device)).copy_transpose([steps, decoder.model_dim]).raw_tensor)
        self.layers = []
        for layer in decoder.layers:
            sa = layer.self_att
            if type(sa) is not CausalSelfAttention or isinstance(sa, (RotaryPosCausalSelfAttention, RelPosCausalSelfAttention)):
                raise TypeError("static decoder step: self-attention %r is not covered" % (sa,))
            if not isinstance(layer.ff, FeedForward):
                raise TypeError("static decoder step: feed-forward %r is not covered" % (layer.ff,))
            H, dk, dv = sa.num_heads.dimension, sa.key_dim_per_head.dimension, sa.value_dim_per_head.dimension
            spec = dict(H=H, dk=dk, dv=dv, sa_norm=_norm(layer.self_att_layer_norm), ff_norm=_norm(layer.ff_layer_norm),
                        qkv=tuple(map(cast, _lin(sa.qkv))), sa_proj=tuple(map(cast, _lin(sa.proj))) if sa.proj else None,
                        ff1=tuple(map(cast, _lin(layer.ff.linear_ff))), ff2=tuple(map(cast, _lin(layer.ff.linear_out))),
                        act=_activation(layer.ff.activation), cross=None)
            if layer.cross_att is not None:
                assert enc is not None and enc_lens is not None, "the decoder has cross-attention: give the encoder output"
                ca = layer.cross_att
                Hc, ck, cv = ca.num_heads.dimension, ca.key_dim_per_head.dimension, ca.value_dim_per_head.dimension
                t_cap = enc.shape[1]
                spec["cross"] = dict(H=Hc, dk=ck, dv=cv, norm=_norm(layer.cross_att_layer_norm), q=tuple(map(cast, _lin(ca.q))),
                                     kv=tuple(map(cast, _lin(ca.kv))), proj=tuple(map(cast, _lin(ca.proj))) if ca.proj else None,
                                     k=torch.zeros(self.num_seqs, Hc, t_cap, ck, dtype=self.dtype, device=self.device),
                                     v=torch.zeros(self.num_seqs, Hc, t_cap, cv, dtype=self.dtype, device=self.device))
            self.layers.append(spec)
        self.final_norm = _norm(decoder.final_layer_norm)
        self.logits_w, self.logits_b = map(cast, _lin(decoder.logits))
        self.enc_capacity = 0
        self._searches = {}
        if enc is not None:
            self.enc_capacity = enc.shape[1]
            self.enc_mask = torch.zeros(self.num_seqs, 1, 1, self.enc_capacity, dtype=torch.bool, device=self.device)
            self.enc_lens = torch.zeros(self.num_seqs, dtype=torch.int32, device=self.device)
            self.set_encoder(enc, enc_lens)
        # static state
        n_layers = len(self.layers)
        first = self.layers[0]
        self.k_cache = torch.zeros(n_layers, num_hyps, first["H"], max_steps, first["dk"], dtype=self.dtype, device=self.device)
        self.v_cache = torch.zeros(n_layers, num_hyps, first["H"], max_steps, first["dv"], dtype=self.dtype, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._steps = torch.arange(max_steps, device=self.device)

    def set_encoder(self, enc: torch.Tensor, enc_lens: torch.Tensor):
        """
        New encoder output for the same object (``[num_seqs, T <= capacity, enc_dim]``): the cross-attention keys / values, lengths and
        the mask are rewritten in place, so captured graphs stay valid.
        """
        t = enc.shape[1]
        assert enc.shape[0] == self.num_seqs and t <= self.enc_capacity, "encoder output %s exceeds the capacity (%i, %i)" % (
            tuple(enc.shape), self.num_seqs, self.enc_capacity)
        x = enc.to(self.dtype)
        for lay in self.layers:
            cr = lay["cross"]
            if cr is None:
                continue
            w, b = cr["kv"]
            kv = F.linear(x, w.t(), b).reshape(self.num_seqs, t, cr["H"], cr["dk"] + cr["dv"])
            cr["k"][:, :, :t].copy_(kv[..., : cr["dk"]].permute(0, 2, 1, 3))
            cr["v"][:, :, :t].copy_(kv[..., cr["dk"]:].permute(0, 2, 1, 3))
        self.enc_lens.copy_(enc_lens.to(self.device, torch.int32))
        self.enc_mask.copy_((torch.arange(self.enc_capacity, device=self.device)[None, :] < self.enc_lens[:, None])[:, None, None, :])

    def reset(self):
        """before a new search over the same encoder output"""
        self.pos.zero_()
        self.k_cache.zero_()
        self.v_cache.zero_()

    def reorder(self, flat: torch.Tensor):
        """hypothesis i continues hypothesis ``flat[i]``: gather the caches along the hypothesis axis (in place)"""
        self.k_cache.copy_(self.k_cache.index_select(1, flat))
        self.v_cache.copy_(self.v_cache.index_select(1, flat))

    def _attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, group: int, lens: Optional[torch.Tensor], mask: torch.Tensor) -> torch.Tensor:
        """
        ``q`` [N, H, d], ``k`` / ``v`` [N / group, H, T, d] -> [N, H * d]. Own kernel for bf16 on the GPU (reads a shared cache once
        per sequence, valid length from ``lens`` or the device step counter); torch's attention otherwise.
        """
        N, H, d = q.shape
        if (q.is_cuda and q.dtype == torch.bfloat16 and d in (64, 128) and v.shape[-1] == d and _lib.use_native(q)
                and hasattr(_lib.get_lib(), "rb200_decode_attention")):
            import ctypes

            q = q.contiguous()
            out = torch.empty(N, H, d, dtype=torch.bfloat16, device=q.device)
            vp, i32 = ctypes.c_void_p, ctypes.c_int
            fn = _lib.bind("rb200_decode_attention", [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, ctypes.c_float, vp, vp])
            _lib.check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr() if lens is not None else None,
                          self.pos.data_ptr() if lens is None else None, N, H, k.shape[2], d, group, float(d) ** -0.5, out.data_ptr(),
                          _lib.stream_ptr()), "decode_attention")
            _lib.count_launch()
            return out.reshape(N, H * d)
        if group > 1:
            k, v, mask = k.repeat_interleave(group, dim=0), v.repeat_interleave(group, dim=0), mask.repeat_interleave(group, dim=0)
        return F.scaled_dot_product_attention(q.unsqueeze(2), k, v, attn_mask=mask).reshape(N, H * v.shape[-1])

    def step(self, prev: torch.Tensor) -> torch.Tensor:
        """``prev`` [N] int64 labels -> logits [N, vocab]; advances the step counter"""
        with torch.autocast(self.device.type, enabled=False):  # the dtype of this object is explicit
            return self._step(prev)

    def _step(self, prev: torch.Tensor) -> torch.Tensor:
        N = self.N
        x = self.emb.index_select(0, prev)
        if self.emb_scale != 1.0:
            x = x * self.emb_scale
        if self.pos_table is not None:
            x = x + self.pos_table.index_select(0, self.pos)  # [1, D] broadcast over hypotheses
        step_mask = (self._steps <= self.pos)[None, None, None, :]  # [1,1,1,L]: positions written so far, incl. this one
        for li, lay in enumerate(self.layers):
            H, dk, dv = lay["H"], lay["dk"], lay["dv"]
            h = _apply_norm(x, lay["sa_norm"])
            w, b = lay["qkv"]
            qkv = F.linear(h, w.t(), b).reshape(N, H, 2 * dk + dv)
            q, k, v = qkv[..., :dk], qkv[..., dk: 2 * dk], qkv[..., 2 * dk:]
            self.k_cache[li].index_copy_(2, self.pos, k.unsqueeze(2))
            self.v_cache[li].index_copy_(2, self.pos, v.unsqueeze(2))
            att = self._attend(q, self.k_cache[li], self.v_cache[li], group=1, lens=None, mask=step_mask)
            if lay["sa_proj"] is not None:
                w, b = lay["sa_proj"]
                att = F.linear(att, w.t(), b)
            x = x + att
            cr = lay["cross"]
            if cr is not None:
                h = _apply_norm(x, cr["norm"])
                w, b = cr["q"]
                q = F.linear(h, w.t(), b).reshape(N, cr["H"], cr["dk"])
                att = self._attend(q, cr["k"], cr["v"], group=self.group, lens=self.enc_lens, mask=self.enc_mask)
                if cr["proj"] is not None:
                    w, b = cr["proj"]
                    att = F.linear(att, w.t(), b)
                x = x + att
            h = _apply_norm(x, lay["ff_norm"])
            w1, b1 = lay["ff1"]
            w2, b2 = lay["ff2"]
            x = x + F.linear(lay["act"](F.linear(h, w1.t(), b1)), w2.t(), b2)
        x = _apply_norm(x, self.final_norm)
        logits = F.linear(x, self.logits_w.t(), self.logits_b)
        self.pos += 1
        return logits


class _Search:
    """buffers and (on CUDA) the captured label step of one search shape; kept on the stepper and reused by later searches"""

    def __init__(self, stepper: StaticTransformerDecoderStep, *, batch: int, beam: int, bos: int, eos: int, use_graph: bool):
        self.stepper, self.batch, self.beam, self.bos, self.eos = stepper, batch, beam, bos, eos
        dev, vocab, L = stepper.device, stepper.vocab, stepper.L
        self.scores = torch.empty(batch, beam, device=dev)
        self.finished = torch.empty(batch, beam, dtype=torch.bool, device=dev)
        self.lengths = torch.empty(batch, beam, dtype=torch.int32, device=dev)
        self.prev = torch.empty(batch * beam, dtype=torch.int64, device=dev)
        self.hist_labels = torch.empty(L, batch, beam, dtype=torch.int32, device=dev)
        self.hist_back = torch.empty(L, batch, beam, dtype=torch.int32, device=dev)
        self.max_len = torch.zeros(batch, dtype=torch.int64, device=dev)
        self._base = torch.arange(batch, device=dev)[:, None] * beam
        self._identity = torch.arange(beam, dtype=torch.int32, device=dev)[None, None, :].expand(L, batch, beam)
        self._forced_row = torch.full((vocab,), float("-inf"), device=dev)  # what a hypothesis at its length limit may score: only eos
        self._forced_row[eos] = 0.0
        self.graph = None
        if use_graph:
            self.reset()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                self.one_label()  # lazy initialisation (library handles, allocator) outside the capture
            torch.cuda.current_stream(dev).wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.one_label()  # (a capture does not run the kernels)

    def reset(self):
        self.stepper.reset()
        self.scores.fill_(float("-inf"))
        self.scores[:, 0] = 0.0
        self.finished.zero_()
        self.lengths.zero_()
        self.prev.fill_(self.bos)
        self.hist_labels.fill_(self.eos)
        self.hist_back.copy_(self._identity)

    def one_label(self):
        st, batch, beam = self.stepper, self.batch, self.beam
        step_idx = st.pos.clone()  # the counter before this label
        logits = st.step(self.prev).reshape(batch, beam, st.vocab).float()
        force_end = (self.lengths >= (self.max_len[:, None] - 1)) & ~self.finished  # at the length limit only eos may follow
        logits = torch.where(force_end[..., None], self._forced_row, logits)
        new_scores, back, lab = seq_ops.beam_topk(logits, self.scores, finished=self.finished, eos=self.eos, k=beam)
        flat = (self._base + back.long()).reshape(-1)
        st.reorder(flat)
        was_finished = self.finished.reshape(-1).index_select(0, flat).reshape(batch, beam)
        self.lengths.copy_(self.lengths.reshape(-1).index_select(0, flat).reshape(batch, beam) + (~was_finished).to(torch.int32))
        self.finished.copy_(was_finished | (lab == self.eos))
        self.scores.copy_(new_scores)
        self.hist_labels.index_copy_(0, step_idx, lab.unsqueeze(0))
        self.hist_back.index_copy_(0, step_idx, back.unsqueeze(0))
        self.prev.copy_(lab.reshape(-1).long())


def beam_search_static(stepper: StaticTransformerDecoderStep, *, batch: int, beam: int, bos: int, eos: int, max_len: torch.Tensor,
                       length_norm: bool = True, use_graph: Optional[bool] = None, check_every: int = 8
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """
    Same search and same return values as :func:`returnn_b200.models.beam_search.beam_search_raw`
    (labels [batch, beam, L] padded with eos, lengths [batch, beam], scores [batch, beam], sorted by score).

    :param max_len: [batch] int (host) longest output per sequence; its maximum must not exceed ``stepper.L``
    :param use_graph: None: on CUDA devices. The search buffers and the captured label step are kept on ``stepper`` and reused by
        later searches with the same (batch, beam, bos, eos); ``stepper.set_encoder`` swaps the encoder output in between.
    :param check_every: the host reads the ``finished`` flags every this many labels
    """
    dev = stepper.device
    vocab = stepper.vocab
    max_steps = int(max_len.max()) if batch else 0
    assert max_steps <= stepper.L and stepper.N == batch * beam
    if use_graph is None:
        use_graph = dev.type == "cuda"
    key = (batch, beam, bos, eos, bool(use_graph))
    search = stepper._searches.get(key)
    if search is None:
        search = stepper._searches[key] = _Search(stepper, batch=batch, beam=beam, bos=bos, eos=eos, use_graph=bool(use_graph) and max_steps > 0)
    search.max_len.copy_(max_len.to(dev))
    search.reset()
    scores, lengths, finished, hist_labels, hist_back = search.scores, search.lengths, search.finished, search.hist_labels, search.hist_back
    n_done = 0
    with torch.no_grad():
        for i in range(max_steps):
            if search.graph is not None:
                search.graph.replay()
            else:
                search.one_label()
            n_done = i + 1
            if (n_done % check_every == 0 or n_done == max_steps) and bool(finished.all()):
                break
    L = n_done
    out = torch.full((batch, beam, max(L, 1)), eos, dtype=torch.int32, device=dev)
    idx = torch.arange(beam, device=dev)[None, :].expand(batch, beam)
    for i in range(L - 1, -1, -1):
        out[:, :, i] = torch.gather(hist_labels[i], 1, idx)
        idx = torch.gather(hist_back[i].long(), 1, idx)
    final = scores.clone()
    if length_norm:
        final = final / torch.clamp(lengths.float(), min=1.0)
    order = torch.argsort(final, dim=1, descending=True)
    return torch.gather(out, 1, order[:, :, None].expand_as(out)), torch.gather(lengths, 1, order), torch.gather(final, 1, order)
