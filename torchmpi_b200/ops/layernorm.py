"""Layer normalisation with a one-pass backward (csrc/kernels/layernorm.cu).

``LayerNorm(C)`` is an ``nn.LayerNorm`` over the last dimension whose CUDA path reads each row once
forward and reads ``(x, dy)`` once backward, producing ``dx``, ``dgamma`` and ``dbeta`` together; eager
PyTorch runs the backward as three kernels.  Inputs the kernel does not cover (CPU, widths that are not
a multiple of 256 bf16 / 128 fp32 elements or above 2048 / 1024, parameters of another dtype) take
``F.layer_norm``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr

launch_count = 0
_scratch = {}


def _scratch_for(dev: torch.device, C: int) -> torch.Tensor:
    key = (dev.index, stream_ptr())
    need = lib.tmpi_layernorm_scratch_bytes(C)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < need:
        buf = _scratch[key] = torch.empty(need, dtype=torch.uint8, device=dev)
    return buf


def supported(x: torch.Tensor, weight, bias) -> bool:
    return (x.is_cuda and weight is not None and bias is not None and weight.dtype == x.dtype and bias.dtype == x.dtype
            and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and has_symbol("tmpi_layernorm_fwd")
            and bool(lib.tmpi_layernorm_supported(x.shape[-1], dtype_code(x.dtype))))


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        global launch_count
        C = x.shape[-1]
        x2 = x.reshape(-1, C).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        check(lib.tmpi_layernorm_fwd(x2.data_ptr(), weight.data_ptr(), bias.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                     rstd.data_ptr(), rows, C, eps, dtype_code(x.dtype), stream_ptr()))
        launch_count += 1
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        global launch_count
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, C = x2.shape
        dy2 = dy.reshape(rows, C).contiguous()
        dx = torch.empty_like(x2)
        dgamma = torch.empty_like(weight)
        dbeta = torch.empty_like(weight)
        check(lib.tmpi_layernorm_bwd(x2.data_ptr(), dy2.data_ptr(), weight.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                     dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), rows, C, dtype_code(x2.dtype),
                                     _scratch_for(x2.device, C).data_ptr(), stream_ptr()))
        launch_count += 2
        return dx.view(ctx.shape), dgamma, dbeta, None


class LayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if len(self.normalized_shape) == 1 and supported(x, self.weight, self.bias):
            return _LayerNormFn.apply(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
