"""Elementwise hot ops: SGD with momentum, EASGD elastic step, Downpour accumulation.

On CUDA tensors each op is one hand-written sm_100a kernel from
csrc/kernels/elementwise.cu (the reference runs several cutorch kernels per op
and tensor: ``w:add(-lr, gw)``, ``old:copy(pref):add(-t); t:add(alpha, old);
old:mul(-alpha)``, ``acc:add(gw)`` - torchmpi/parameterserver/easgdupdate.lua:73-75,
torchmpi/parameterserver/downpourupdate.lua:49-59).  CPU tensors take the same
arithmetic in PyTorch.  A CUDA tensor never falls back silently: a missing
kernel raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr


def _need(sym: str) -> None:
    if not has_symbol(sym):
        raise RuntimeError(f"torchmpi_b200: native kernel '{sym}' is missing from libtorchmpi_b200.so")


def easgd_elastic(local: torch.Tensor, center: torch.Tensor, delta: torch.Tensor, alpha: float) -> None:
    """``d = center - local; local += alpha * d; delta = -alpha * d`` in one pass."""
    if local.is_cuda:
        _need("tmpi_easgd_elastic")
        c = center if center.is_cuda else center.to(local.device, non_blocking=True)
        assert local.is_contiguous() and c.is_contiguous() and delta.is_contiguous()
        check(lib.tmpi_easgd_elastic(local.data_ptr(), c.data_ptr(), delta.data_ptr(), local.numel(),
                                     dtype_code(local.dtype), float(alpha), stream_ptr()))
        return
    with torch.no_grad():
        d = center.to(local.dtype) - local
        local.add_(d, alpha=alpha)
        delta.copy_(d).mul_(-alpha)


def downpour_accum(accum: torch.Tensor, grad: torch.Tensor, scale: float = 1.0, zero_first: bool = False) -> None:
    """``accum = (0 if zero_first else accum) + scale * grad``."""
    if accum.is_cuda:
        _need("tmpi_downpour_accum")
        assert accum.is_contiguous() and grad.is_contiguous() and accum.dtype == grad.dtype
        check(lib.tmpi_downpour_accum(accum.data_ptr(), grad.data_ptr(), accum.numel(), dtype_code(accum.dtype),
                                      float(scale), 1 if zero_first else 0, stream_ptr()))
        return
    with torch.no_grad():
        if zero_first:
            accum.zero_()
        accum.add_(grad, alpha=scale)


def sgd_momentum_(weight: torch.Tensor, grad: torch.Tensor, *, lr: float, momentum: float = 0.0,
                  dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False,
                  grad_scale: float = 1.0, master: Optional[torch.Tensor] = None,
                  momentum_buf: Optional[torch.Tensor] = None, first_step: bool = False,
                  zero_grad: bool = False) -> None:
    """One fused SGD step on a flat tensor (torch.optim.SGD arithmetic).

    ``master`` (fp32) holds the true weights when ``weight`` is bf16/fp16; ``momentum_buf`` is fp32.
    """
    if weight.is_cuda:
        _need("tmpi_sgd_momentum")
        check(lib.tmpi_sgd_momentum(
            weight.data_ptr(), dtype_code(weight.dtype), grad.data_ptr(), dtype_code(grad.dtype),
            master.data_ptr() if master is not None else None,
            momentum_buf.data_ptr() if momentum_buf is not None else None,
            weight.numel(), lr, momentum, dampening, weight_decay, grad_scale,
            1 if nesterov else 0, 1 if first_step else 0, 1 if zero_grad else 0, stream_ptr()))
        return
    with torch.no_grad():
        w = master if master is not None else weight
        g = grad.to(torch.float32) * grad_scale if w.dtype == torch.float32 else grad * grad_scale
        if weight_decay:
            g = g + weight_decay * w
        if momentum_buf is not None and momentum != 0.0:
            if first_step:
                momentum_buf.copy_(g)
            else:
                momentum_buf.mul_(momentum).add_(g, alpha=1 - dampening)
            g = g + momentum * momentum_buf if nesterov else momentum_buf
        w.add_(g.to(w.dtype), alpha=-lr)
        if master is not None:
            weight.copy_(master)
        if zero_grad:
            grad.zero_()
