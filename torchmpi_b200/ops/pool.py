"""Max pooling for channels-last activations (csrc/kernels/pool.cu).

``MaxPool2d(k, stride, padding)`` keeps a one-byte window index per output element, so backward is
a gather that writes every gradient byte once.  CPU tensors, other layouts and channel counts that
do not fill 16-byte packs take ``torch.nn.functional.max_pool2d``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr

launch_count = 0


def supported(x: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dim() == 4 and has_symbol("tmpi_maxpool_fwd")):
        return False
    if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return False
    return x.shape[1] % (16 // x.element_size()) == 0


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, s, p):
        global launch_count
        x = x.contiguous(memory_format=torch.channels_last)
        N, C, H, W = x.shape
        OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((N, OH, OW, C), dtype=torch.uint8, device=x.device)
        check(lib.tmpi_maxpool_fwd(x.data_ptr(), y.data_ptr(), idx.data_ptr(), N, H, W, C, OH, OW, k, s, p,
                                   dtype_code(x.dtype), stream_ptr()))
        launch_count += 1
        ctx.save_for_backward(idx)
        ctx.dims = (N, H, W, C, OH, OW, k, s, p)
        return y

    @staticmethod
    def backward(ctx, dy):
        global launch_count
        (idx,) = ctx.saved_tensors
        N, H, W, C, OH, OW, k, s, p = ctx.dims
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty((N, C, H, W), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        check(lib.tmpi_maxpool_bwd(dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), N, H, W, C, OH, OW, k, s, p,
                                   dtype_code(dy.dtype), stream_ptr()))
        launch_count += 1
        return dx, None, None, None


class MaxPool2d(nn.Module):
    def __init__(self, kernel_size: int, stride: int = None, padding: int = 0):
        super().__init__()
        self.k, self.s, self.p = kernel_size, stride or kernel_size, padding

    def forward(self, x):
        if supported(x) and self.p < self.k:
            return _MaxPoolFn.apply(x, self.k, self.s, self.p)
        return F.max_pool2d(x, self.k, self.s, self.p)
