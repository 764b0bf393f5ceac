"""The ResNet stem (7x7, stride 2, pad 3, 3 input channels) as im2col + tcgen05 GEMM.

``StemConv7x7`` is an ``nn.Conv2d(3, C, 7, stride=2, padding=3, bias=False)`` with the same parameter
(``weight [C, 3, 7, 7]``), so checkpoints and parameter counts do not change.  On a channels-last
bf16 CUDA input, forward writes the patch matrix ``col [N*OH*OW, 160]`` with one kernel
(csrc/kernels/im2col.cu) and multiplies it with the ``[C, 160]`` weight matrix on the tensor cores;
the result is the channels-last output as it lies.  Backward needs only the weight gradient (the
image has none): ``dW = dY^T col``, a split-K product on the same tensor-core kernel family over the saved
patch matrix.  Other inputs take
``F.conv2d``.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr
from . import gemm

launch_count = 0
PATCH = 147


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dim() == 4 and x.shape[1] == 3 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and tuple(w.shape[1:]) == (3, 7, 7) and w.shape[0] % 8 == 0 and (x.shape[3] * 3 * 2) % 16 == 0
            and x.is_contiguous(memory_format=torch.channels_last) and not x.requires_grad
            and has_symbol("tmpi_stem_im2col") and has_symbol("tmpi_gemm_bf16"))


class _StemConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        global launch_count
        N, _, H, W = x.shape
        OH, OW = (H + 6 - 7) // 2 + 1, (W + 6 - 7) // 2 + 1
        M, Cout = N * OH * OW, w.shape[0]
        kpad = lib.tmpi_stem_patch_width()
        col = torch.empty((M, kpad), dtype=x.dtype, device=x.device)
        check(lib.tmpi_stem_im2col(x.data_ptr(), col.data_ptr(), N, H, W, dtype_code(x.dtype), stream_ptr()))
        w2d = torch.zeros((Cout, kpad), dtype=w.dtype, device=w.device)
        w2d[:, :PATCH] = w.permute(0, 2, 3, 1).reshape(Cout, PATCH)          # (kh, kw, c) order of the patch rows
        y = torch.empty((N, Cout, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        gemm.matmul_nt(col, w2d, out=y.permute(0, 2, 3, 1).reshape(M, Cout))
        launch_count += 2
        ctx.save_for_backward(col)
        ctx.wshape = tuple(w.shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        (col,) = ctx.saved_tensors
        Cout = ctx.wshape[0]
        dy2d = dy.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1).reshape(-1, Cout)
        from .conv import matmul_tn_splitk
        dw2d = matmul_tn_splitk(dy2d, col)                                   # [Cout, 160]: split over the 3.2 M patch rows
        dw = dw2d[:, :PATCH].reshape(Cout, 7, 7, 3).permute(0, 3, 1, 2)
        return None, dw


class StemConv7x7(nn.Conv2d):
    def __init__(self, out_channels: int):
        super().__init__(3, out_channels, 7, stride=2, padding=3, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if supported(x, self.weight):
            return _StemConvFn.apply(x, self.weight)
        return F.conv2d(x, self.weight, None, self.stride, self.padding)
