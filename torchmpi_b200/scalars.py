"""Scalar collectives and the replicated-value sanity check.

``allreduce_<T>(v)``, ``broadcast_<T>(root, v)``, ``reduce_<T>(root, v)`` and
``sendreceive_<T>(v, src, dst)`` for the seven C types of the reference
(torchmpi/init.lua:125-134) act on the communicator under the *cursor* (not on
the collective span), like lib/collectives.cpp:38-59.  ``reduce_<T>`` is declared
but never compiled in the reference (lib/collectives.cpp:615-620); it works here.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import runtime
from . import gdist
from .runtime import S

_TYPES = {"uint8_t": torch.uint8, "char": torch.int8, "short": torch.int16, "int": torch.int32,
          "long": torch.int64, "float": torch.float32, "double": torch.float64}

__all__ = []


def _group():
    runtime._require_started()
    members = runtime.current_members()
    return members, runtime.group_for(members)


def _py(t: torch.Tensor):
    return t.item()


def _mk(tname: str, dt: torch.dtype):
    def allreduce(v):
        members, g = _group()
        t = torch.tensor([v], dtype=dt)
        if g is not None:
            gdist.all_reduce(t, g)
        return _py(t)

    def broadcast(root, v):
        members, g = _group()
        t = torch.tensor([v], dtype=dt)
        if g is not None:
            gdist.broadcast(t, members[root], g)
        return _py(t)

    def reduce(root, v):
        members, g = _group()
        t = torch.tensor([v], dtype=dt)
        if g is not None:
            gdist.reduce(t, members[root], g)
        return _py(t) if members[root] == S.rank else v

    def sendreceive(v, src, dst):
        members, g = _group()
        me = members.index(S.rank)
        if g is None or (src == me and dst == me):
            return v
        t, r = torch.tensor([v], dtype=dt), torch.zeros(1, dtype=dt)
        gdist.sendrecv(t, r, members[dst], members[src], g)
        return _py(r)

    for op, fn in (("allreduce", allreduce), ("broadcast", broadcast), ("reduce", reduce), ("sendreceive", sendreceive)):
        name = f"{op}_{tname}"
        fn.__name__ = name
        globals()[name] = fn
        __all__.append(name)


for _n, _d in _TYPES.items():
    _mk(_n, _d)


def abs_mean_var(t: torch.Tensor):
    """(mean(|t|), unbiased var(|t|)) in float64; one fused pass on the GPU when the kernel is there."""
    if t.is_cuda:
        from .ops import stats
        return stats.absmean_var(t)
    a = t.detach().double().abs()
    return a.mean().item(), (a.var().item() if a.numel() > 1 else 0.0)


def check_with_allreduce(inp, name: str = "", tol: float = 1e-7) -> None:
    """Asserts that a replicated quantity is the same on every rank of the current communicator.

    Compares this rank's abs-mean and abs-variance with their averages over the
    ranks, relative tolerance 1e-7 (torchmpi/init.lua:372-395).
    """
    n = runtime.size()
    if isinstance(inp, torch.Tensor):
        m, v = abs_mean_var(inp)
    else:
        m = v = abs(float(inp))
    m_sync = globals()["allreduce_double"](m) / n
    v_sync = globals()["allreduce_double"](v) / n
    if not ((m == 0 and m_sync == 0) or abs((m - m_sync) / (m if m != 0 else 1.0)) < tol):
        raise AssertionError(f"{name}: absmean {m} vs absmean_sync {m_sync}")
    if not ((v == 0 and v_sync == 0) or abs((v - v_sync) / (v if v != 0 else 1.0)) < tol):
        raise AssertionError(f"{name}: absvar {v} vs absvar_sync {v_sync}")


__all__ += ["check_with_allreduce", "abs_mean_var"]
