"""abs-mean / abs-variance of a tensor in one pass (the oracle of ``check_with_allreduce``).

The reference computes ``input:float():clone():abs():mean()`` and ``:var()``
separately (torchmpi/init.lua:372-381): several temporaries and passes.  The
CUDA kernel reads the tensor once and reduces sum |x| and sum x^2 in fp64.
"""
from __future__ import annotations

import ctypes as C

import torch

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr

_scratch = {}


def absmean_var(t: torch.Tensor):
    """(mean(|t|), unbiased variance of |t|) as Python floats."""
    n = t.numel()
    if n == 0:
        return 0.0, 0.0
    if not t.is_cuda:
        a = t.detach().double().abs()
        return a.mean().item(), (a.var().item() if n > 1 else 0.0)
    if not has_symbol("tmpi_absmean_var"):
        raise RuntimeError("torchmpi_b200: native kernel 'tmpi_absmean_var' is missing")
    t = t.contiguous()
    dev = t.device
    key = dev.index
    if key not in _scratch:
        _scratch[key] = (torch.zeros(lib.tmpi_absmean_var_scratch_bytes(), dtype=torch.uint8, device=dev),
                         torch.empty(2, dtype=torch.float64, device=dev))
    scratch, out = _scratch[key]
    check(lib.tmpi_absmean_var(t.data_ptr(), dtype_code(t.dtype), n, out.data_ptr(), scratch.data_ptr(), stream_ptr()))
    s1, s2 = out.tolist()
    mean = s1 / n
    var = max(0.0, (s2 - n * mean * mean) / (n - 1)) if n > 1 else 0.0
    return mean, var
