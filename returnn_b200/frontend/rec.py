"""
Recurrent layers: ``LSTM`` and ``ZoneoutLSTM``.

Parameter layout (checkpoint compatible): ``ff_weight [4*out, in]``, ``rec_weight [4*out, out]``, ``bias [4*out]``,
gate order i, f, g (cell input), o. Frames beyond a sequence's length produce zeros and do not touch the state,
so the final state is the state after the last valid frame.

Execution goes through :mod:`returnn_b200.ops.lstm`: on B200 a persistent kernel keeps the recurrent matrix resident in
shared memory across the SMs for the whole sequence; on CPU the packed-sequence LSTM of torch is used.

Parity: returnn/frontend/rec.py:17-130; returnn/torch/frontend/_backend.py:2718-2850; cell math
returnn/native_op.py:1082-1179.
"""

from __future__ import annotations
from typing import Optional, Sequence, Tuple
import torch
from ..tensor import Tensor, Dim, single_step_dim, batch_dim
from .module import Module
from .parameter import Parameter
from .state import State
from . import init as _init
from ._utils import wrap

__all__ = ["LSTM", "LstmState", "ZoneoutLSTM", "bidirectional_lstm"]


class LstmState(State):
    """h and c"""

    def __init__(self, *_args, h: Tensor = None, c: Tensor = None):
        super().__init__(*_args)
        if not _args:
            self.h = h
            self.c = c


class LSTM(Module):
    """single-direction LSTM over a spatial dim, or one step with ``spatial_dim=single_step_dim``"""

    def __init__(self, in_dim: Dim, out_dim: Dim, *, with_bias: bool = True):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.ff_weight = Parameter((4 * self.out_dim, self.in_dim))
        self.ff_weight.initial = _init.Glorot()
        self.rec_weight = Parameter((4 * self.out_dim, self.out_dim))
        self.rec_weight.initial = _init.Glorot()
        self.bias = None
        if with_bias:
            self.bias = Parameter((4 * self.out_dim,))
            self.bias.initial = 0.0

    def __call__(self, source: Tensor, *, state: LstmState, spatial_dim: Dim, direction: int = 1) -> Tuple[Tensor, LstmState]:
        """
        :param source: {batch.., spatial_dim, in_dim}
        :param state: initial h, c {batch.., out_dim}
        :param direction: +1 forward in time, -1 backward (each sequence reversed within its own length)
        :return: output {spatial_dim, batch.., out_dim}, final state
        """
        if state.h is None or state.c is None:
            raise ValueError("%s: state.h and state.c need to be set (use default_initial_state)" % self)
        if self.in_dim not in source.dims:
            raise ValueError("%s: input %r does not have in_dim %r" % (self, source, self.in_dim))
        from ..ops import lstm as _lstm

        single = spatial_dim == single_step_dim
        bdims = [d for d in source.dims if d not in (spatial_dim, self.in_dim)]
        if single:
            x = source.copy_compatible_to_dims_raw(bdims + [self.in_dim]).unsqueeze(0)
        else:
            x = source.copy_compatible_to_dims_raw([spatial_dim] + bdims + [self.in_dim])
        T = x.shape[0]
        bshape = list(x.shape[1:-1])
        x = x.reshape(T, -1, x.shape[-1])
        B = x.shape[1]
        h0 = state.h.copy_compatible_to_dims_raw(bdims + [self.out_dim]).expand(*bshape, -1).reshape(B, -1)
        c0 = state.c.copy_compatible_to_dims_raw(bdims + [self.out_dim]).expand(*bshape, -1).reshape(B, -1)
        lens = None
        if not single and spatial_dim.is_dynamic() and spatial_dim.dyn_size_ext is not None and spatial_dim.dyn_size_ext.dims:
            sz = spatial_dim.dyn_size_ext
            if all(d in bdims for d in sz.dims):
                lens = sz.copy_compatible_to_dims_raw(bdims).expand(*bshape).reshape(B).to(torch.int32)
        y, hT, cT = _lstm.lstm(x, lens, self.ff_weight.raw_tensor, self.rec_weight.raw_tensor,
                               self.bias.raw_tensor if self.bias is not None else None, h0, c0, reverse=direction < 0)
        new_state = LstmState(h=wrap(hT.reshape(bshape + [-1]), bdims + [self.out_dim], feature_dim=self.out_dim),
                              c=wrap(cT.reshape(bshape + [-1]), bdims + [self.out_dim], feature_dim=self.out_dim))
        if single:
            out = wrap(y.reshape(bshape + [-1]), bdims + [self.out_dim], feature_dim=self.out_dim)
        else:
            out = wrap(y.reshape([T] + bshape + [-1]), [spatial_dim] + bdims + [self.out_dim], feature_dim=self.out_dim)
        return out, new_state

    def default_initial_state(self, *, batch_dims: Sequence[Dim]) -> LstmState:
        """zeros"""
        from .const import zeros

        return LstmState(h=zeros(list(batch_dims) + [self.out_dim], feature_dim=self.out_dim),
                         c=zeros(list(batch_dims) + [self.out_dim], feature_dim=self.out_dim))


def bidirectional_lstm(fw: LSTM, bw: LSTM, source: Tensor, *, spatial_dim: Dim, state_fw: Optional[LstmState] = None,
                       state_bw: Optional[LstmState] = None) -> Tuple[Tensor, Tensor, LstmState, LstmState]:
    """
    ``fw(source, direction=1)`` and ``bw(source, direction=-1)`` over the same input. Same results as the two calls; on the GPU
    both time loops run in one persistent kernel when the sizes agree (see ``ops.lstm.blstm``).

    :return: output of fw, output of bw ({spatial_dim, batch.., out_dim} each), final states of fw and bw
    """
    from ..ops import lstm as _lstm

    bdims = [d for d in source.dims if d not in (spatial_dim, fw.in_dim)]
    if state_fw is None:
        state_fw = fw.default_initial_state(batch_dims=bdims)
    if state_bw is None:
        state_bw = bw.default_initial_state(batch_dims=bdims)
    fusable = (type(fw) is LSTM and type(bw) is LSTM and fw.in_dim == bw.in_dim and fw.out_dim.dimension == bw.out_dim.dimension
               and spatial_dim != single_step_dim and source.raw_tensor.is_cuda and (fw.bias is None) == (bw.bias is None))
    if not fusable:
        yf, sf = fw(source, state=state_fw, spatial_dim=spatial_dim, direction=1)
        yb, sb = bw(source, state=state_bw, spatial_dim=spatial_dim, direction=-1)
        return yf, yb, sf, sb
    x = source.copy_compatible_to_dims_raw([spatial_dim] + bdims + [fw.in_dim])
    T = x.shape[0]
    bshape = list(x.shape[1:-1])
    x = x.reshape(T, -1, x.shape[-1])
    B = x.shape[1]

    def flat(t: Tensor, out_dim: Dim):
        return t.copy_compatible_to_dims_raw(bdims + [out_dim]).expand(*bshape, -1).reshape(B, -1)

    lens = None
    if spatial_dim.is_dynamic() and spatial_dim.dyn_size_ext is not None and spatial_dim.dyn_size_ext.dims:
        sz = spatial_dim.dyn_size_ext
        if all(d in bdims for d in sz.dims):
            lens = sz.copy_compatible_to_dims_raw(bdims).expand(*bshape).reshape(B).to(torch.int32)
    params = [(m.ff_weight.raw_tensor, m.rec_weight.raw_tensor, m.bias.raw_tensor if m.bias is not None else None) for m in (fw, bw)]
    (yf, hf, cf), (yb, hb, cb) = _lstm.blstm(x, lens, params[0], params[1], flat(state_fw.h, fw.out_dim), flat(state_fw.c, fw.out_dim),
                                             flat(state_bw.h, bw.out_dim), flat(state_bw.c, bw.out_dim))
    res = []
    for m, y, h, c in ((fw, yf, hf, cf), (bw, yb, hb, cb)):
        st = LstmState(h=wrap(h.reshape(bshape + [-1]), bdims + [m.out_dim], feature_dim=m.out_dim),
                       c=wrap(c.reshape(bshape + [-1]), bdims + [m.out_dim], feature_dim=m.out_dim))
        res.append((wrap(y.reshape([T] + bshape + [-1]), [spatial_dim] + bdims + [m.out_dim], feature_dim=m.out_dim), st))
    return res[0][0], res[1][0], res[0][1], res[1][1]


class ZoneoutLSTM(LSTM):
    """
    LSTM with zoneout: in training each unit keeps its previous h (c) with probability zoneout_factor_output
    (zoneout_factor_cell); in eval the expectation is used.
    """

    def __init__(self, in_dim: Dim, out_dim: Dim, *, with_bias: bool = True, zoneout_factor_cell: float = 0.0,
                 zoneout_factor_output: float = 0.0, use_zoneout_output: bool = True, forget_bias: float = 0.0,
                 parts_order: str = "ifco"):
        super().__init__(in_dim, out_dim, with_bias=with_bias)
        self.zoneout_factor_cell = zoneout_factor_cell
        self.zoneout_factor_output = zoneout_factor_output
        self.use_zoneout_output = use_zoneout_output
        self.forget_bias = forget_bias
        parts_order = parts_order.replace("c", "j").replace("g", "j")
        assert len(parts_order) == 4 and set(parts_order) == set("ijfo"), "invalid parts_order"
        self.parts_order = parts_order

    def __call__(self, source: Tensor, *, state: LstmState, spatial_dim: Dim) -> Tuple[Tensor, LstmState]:
        from .run_ctx import get_run_ctx
        from .loop import scan

        if spatial_dim == single_step_dim:
            return self._step(source, state)
        out, last, _ = scan(spatial_dim=spatial_dim, xs=source, ys=None, initial=state,
                            body=lambda x, s: self._step(x, s))
        return out, last

    def _step(self, x: Tensor, state: LstmState) -> Tuple[Tensor, LstmState]:
        from .run_ctx import get_run_ctx

        bdims = [d for d in x.dims if d != self.in_dim]
        xr = x.copy_compatible_to_dims_raw(bdims + [self.in_dim])
        h = state.h.copy_compatible_to_dims_raw(bdims + [self.out_dim])
        c = state.c.copy_compatible_to_dims_raw(bdims + [self.out_dim])
        z = torch.nn.functional.linear(xr, self.ff_weight.raw_tensor) + torch.nn.functional.linear(h, self.rec_weight.raw_tensor)
        if self.bias is not None:
            z = z + self.bias.raw_tensor
        parts = dict(zip(self.parts_order, torch.chunk(z, 4, dim=-1)))
        i, j, f, o = parts["i"], parts["j"], parts["f"], parts["o"]
        new_c = torch.sigmoid(f + self.forget_bias) * c + torch.sigmoid(i) * torch.tanh(j)
        new_h = torch.sigmoid(o) * torch.tanh(new_c)
        train = get_run_ctx().is_train_flag_enabled(func=ZoneoutLSTM.__call__)
        train = bool(train.raw_tensor) if isinstance(train, Tensor) else bool(train)

        def zone(new, old, p):
            if not p:
                return new
            if train:
                keep_new = torch.empty_like(new).bernoulli_(1.0 - p)
                return keep_new * new + (1.0 - keep_new) * old
            return (1.0 - p) * new + p * old

        out_c = zone(new_c, c, self.zoneout_factor_cell)
        out_h = zone(new_h, h, self.zoneout_factor_output)
        y = out_h if self.use_zoneout_output else new_h
        ns = LstmState(h=wrap(out_h, bdims + [self.out_dim], feature_dim=self.out_dim),
                       c=wrap(out_c, bdims + [self.out_dim], feature_dim=self.out_dim))
        return wrap(y, bdims + [self.out_dim], feature_dim=self.out_dim), ns
