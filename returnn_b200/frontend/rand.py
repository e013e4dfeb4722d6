"""
Random numbers. One global torch generator per device, seeded by ``set_random_seed``; ``static=True`` draws
(parameter init) and dynamic draws (dropout, sampling) use separate generators so that adding a dropout call does
not change the initial weights.

Parity: returnn/frontend/rand.py (set_random_seed, get_random_state, random, random_uniform/normal/truncated_normal).
"""

from __future__ import annotations
from typing import Dict, Optional, Sequence, Union
import numpy
import torch
from ..tensor import Tensor, Dim
from ._utils import wrap, torch_dtype, shape_of, get_default_float_dtype

__all__ = ["set_random_seed", "get_random_state", "set_random_state", "reset_rng_states", "random", "random_uniform",
           "random_normal", "random_truncated_normal", "random_choice_without_replacement", "random_choice_with_replacement", "random_label",
           "reset_step_random_state", "get_static_step_based_seed"]

_seed = 42
_gens: Dict[str, torch.Generator] = {}


def set_random_seed(seed: int):
    """seed all generators"""
    global _seed
    _seed = int(seed)
    _gens.clear()
    torch.manual_seed(_seed)


def _gen(device, static: bool) -> torch.Generator:
    dev = torch.device(device or "cpu")
    key = "%s/%s" % (dev, "static" if static else "dyn")
    g = _gens.get(key)
    if g is None:
        g = torch.Generator(device=dev)
        g.manual_seed((_seed * 2 + (1 if static else 0)) % (2**63))
        _gens[key] = g
    return g


def get_random_state() -> Dict[str, bytes]:
    """states of all generators"""
    return {k: g.get_state() for k, g in _gens.items()}


def set_random_state(state: Dict[str, bytes]):
    """restore"""
    for k, s in state.items():
        if k in _gens:
            _gens[k].set_state(s)


def reset_rng_states():
    """forget generators (re-created from the seed)"""
    _gens.clear()


def random(*, dims: Sequence[Dim], dtype: Optional[str] = None, device: Optional[str] = None,
           sparse_dim: Optional[Dim] = None, feature_dim: Optional[Dim] = None, distribution: str,
           mean=None, stddev=None, bound=None, minval=None, maxval=None, seed=None, algorithm=None,
           explicit_state=None, auto_update_state=None, static: Optional[bool] = None, out: Optional[Tensor] = None) -> Tensor:
    """
    :param distribution: uniform / normal / truncated_normal
    :param static: draw for parameter init
    """
    if dtype is None:
        dtype = get_default_float_dtype()
    if device is None:
        from .device import get_default_device

        device = get_default_device()
    shape = shape_of(dims)
    tdt = torch_dtype(dtype)
    from . import _random_journal

    journal, journal_mode = _random_journal.current_journal()
    if journal_mode == "replay":  # the draw recorded by another run takes the place of this one
        entry = journal.get_next(shape=shape, dtype=dtype, distribution=distribution)
        raw = torch.from_numpy(entry.out).to(device=device, dtype=tdt)
        res = wrap(raw, dims, sparse_dim=sparse_dim, feature_dim=feature_dim)
        if out is not None:
            out.raw_tensor = raw
            return out
        return res
    g = _gen(device, bool(static))
    if seed is not None:
        g = torch.Generator(device=torch.device(device or "cpu"))
        g.manual_seed(int(seed))
    gen_dt = tdt if tdt in (torch.float32, torch.float64) or not tdt.is_floating_point else torch.float32
    if distribution == "uniform":
        if bound is not None:
            minval, maxval = -bound, bound
        if minval is None:
            minval = 0
        if maxval is None:
            maxval = 1
        if tdt.is_floating_point:
            raw = torch.empty(shape, dtype=gen_dt, device=device).uniform_(float(_v(minval)), float(_v(maxval)), generator=g)
        else:
            raw = torch.randint(int(_v(minval)), int(_v(maxval)), shape, dtype=tdt, device=device, generator=g)
    elif distribution == "normal":
        raw = torch.empty(shape, dtype=gen_dt, device=device).normal_(float(_v(mean) or 0.0), float(_v(stddev) if stddev is not None else 1.0), generator=g)
    elif distribution == "truncated_normal":
        m = float(_v(mean) or 0.0)
        s = float(_v(stddev) if stddev is not None else 1.0)
        raw = torch.empty(shape, dtype=gen_dt, device=device)
        torch.nn.init.trunc_normal_(raw, mean=m, std=s, a=m - 2 * s, b=m + 2 * s, generator=g)
    else:
        raise ValueError("random: invalid distribution %r" % distribution)
    if raw.dtype != tdt:
        raw = raw.to(tdt)
    if journal_mode == "record":
        journal.append(out=(raw.float() if raw.dtype == torch.bfloat16 else raw).detach().cpu().numpy(), dtype=dtype, distribution=distribution,
                       mean=mean, stddev=stddev, bound=bound, minval=minval, maxval=maxval, seed=seed, static=static)
    res = wrap(raw, dims, sparse_dim=sparse_dim, feature_dim=feature_dim)
    if out is not None:
        out.raw_tensor = raw
        return out
    return res


def _v(x):
    if isinstance(x, Tensor):
        return x._raw_tensor.item()
    return x


def random_uniform(dims, *, dtype=None, device=None, sparse_dim=None, feature_dim=None, minval=0, maxval=1, seed=None, static=None, **_kw):
    """uniform"""
    return random(dims=dims, dtype=dtype, device=device, sparse_dim=sparse_dim, feature_dim=feature_dim,
                  distribution="uniform", minval=minval, maxval=maxval, seed=seed, static=static)


def random_normal(dims, *, dtype=None, device=None, sparse_dim=None, feature_dim=None, mean=0.0, stddev=1.0, seed=None, static=None, **_kw):
    """normal"""
    return random(dims=dims, dtype=dtype, device=device, sparse_dim=sparse_dim, feature_dim=feature_dim,
                  distribution="normal", mean=mean, stddev=stddev, seed=seed, static=static)


def random_truncated_normal(dims, *, dtype=None, device=None, sparse_dim=None, feature_dim=None, mean=0.0, stddev=1.0, seed=None, static=None, **_kw):
    """normal truncated at 2 stddev"""
    return random(dims=dims, dtype=dtype, device=device, sparse_dim=sparse_dim, feature_dim=feature_dim,
                  distribution="truncated_normal", mean=mean, stddev=stddev, seed=seed, static=static)


def random_choice_with_replacement(dims: Sequence[Dim], *, probs: Tensor, axis: Dim) -> Tensor:
    """sample indices of axis from probs; result has dims + probs' other dims"""
    from ._utils import axis_of

    rest = [d for d in probs.dims if d != axis]
    extra = [d for d in dims if d not in rest]
    praw = probs.copy_compatible_to_dims_raw(rest + [axis])
    n = 1
    for d in extra:
        n *= d.get_dim_value()
    flat = praw.reshape(-1, praw.shape[-1]).float()
    idx = torch.multinomial(flat, n, replacement=True, generator=_gen(str(flat.device), False))
    idx = idx.reshape(list(praw.shape[:-1]) + [d.get_dim_value() for d in extra]).to(torch.int32)
    return wrap(idx, rest + extra, sparse_dim=axis)


def random_choice_without_replacement(*, log_probs: Tensor, axis: Dim, k: Union[int, Dim]) -> Tensor:
    """Gumbel top-k sampling without replacement"""
    from .reduce import top_k

    g = random(dims=log_probs.dims, dtype=log_probs.dtype, device=log_probs.device, distribution="uniform", minval=1e-20, maxval=1.0)
    gumbel = wrap(-torch.log(-torch.log(g._raw_tensor)), log_probs.dims)
    k_dim = k if isinstance(k, Dim) else Dim(k, name="random-choice-k")
    _, idx, _ = top_k(log_probs + gumbel, axis=axis, k_dim=k_dim)
    return idx


def random_label(dims: Sequence[Dim], sparse_dim: Dim, *, dtype: str = "int32", device=None) -> Tensor:
    """uniform random class indices"""
    return random(dims=dims, dtype=dtype, device=device, sparse_dim=sparse_dim, distribution="uniform", minval=0, maxval=sparse_dim.dimension)


# seeds for ``random(..., static=True)``: a host random state that is rewound at the start of every step, so that the n-th static
# random call of a step gets the same seed in every step (and in the forward and the recomputation of a checkpointed region)
_step_rnd_seed = 42
_step_rnd = numpy.random.RandomState(_step_rnd_seed)


def reset_step_random_state():
    """rewind the step-based seed sequence; called at the beginning of every step"""
    _step_rnd.seed(_step_rnd_seed)


def get_static_step_based_seed(*, size=None):
    """the next seed (or array of seeds) of the step-based sequence"""
    return _step_rnd.randint(2 ** 31, size=size)
