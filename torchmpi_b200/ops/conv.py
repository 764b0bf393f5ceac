"""Convolutions of channels-last bf16 activations on the hand-written implicit-GEMM kernel
(csrc/kernels/conv_gemm.cu): forward, input gradient and weight gradient read the activation through
TMA (plain tiles for 1x1 / stride 1, im2col-mode loads otherwise) and the weight as it lies in a
channels-last ``Conv2d`` parameter; no patch matrix and no transposed copy is written.

``conv2d(x, w, stride, padding)`` is the autograd op.  ``conv2d_bn_stats`` also returns the per-CTA partial
sums of the output's batch statistics, which ``ops.bn_relu`` consumes in place of its own statistics pass
(``ConvBnReLU`` below ties the two together).  ``fuse_add`` lets the input gradient absorb a second gradient
that flows into the same activation (the identity branch of a residual block), replacing autograd's
accumulation kernel.  Shapes the kernel does not take (channels not a multiple of 64, strided input
gradients, other dtypes, CPU) fall back to ``F.conv2d``.  The reference has no convolution at all.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .._lib import lib, check, has_symbol, stream_ptr, TorchMPIError

launch_count = 0
_ws = {}


def _workspace(dev: torch.device, need: int) -> torch.Tensor:
    """Per (device, stream) workspace for the fp32 partial tiles of the weight gradient."""
    key = (dev.index, stream_ptr())
    buf = _ws.get(key)
    if buf is None or buf.numel() < need:
        buf = _ws[key] = torch.empty(max(need, 64 << 20), dtype=torch.uint8, device=dev)
    return buf


def supported(x: torch.Tensor, w: torch.Tensor, stride: int, padding: int) -> bool:
    if not (has_symbol("tmpi_conv_fwd") and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        return False
    Cout, Cin, R, S = w.shape
    return (Cin % 64 == 0 and Cout % 64 == 0 and R == S and padding <= R - 1 and x.shape[1] == Cin
            and x.shape[0] * x.shape[2] * x.shape[3] < 2 ** 31)


def _cl(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous(memory_format=torch.channels_last) else t.contiguous(memory_format=torch.channels_last)


def _out_hw(H, W, R, S, stride, pad):
    return (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1


def conv_forward(x, w, stride, pad, stats: Optional[torch.Tensor] = None):
    """Raw forward launch: returns ``(y, stat_rows)``; ``stats`` (fp32, at least ``max_ctas * 2 * Cout``) receives
    the partial sums when given."""
    global launch_count
    N, Cin, H, W = x.shape
    Cout, _, R, S = w.shape
    Ho, Wo = _out_hw(H, W, R, S, stride, pad)
    y = torch.empty((N, Cout, Ho, Wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    rows = C.c_int(0)
    check(lib.tmpi_conv_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), N, H, W, Cin, Cout, R, S, stride, pad,
                            stats.data_ptr() if stats is not None else None, C.byref(rows), stream_ptr()))
    launch_count += 1
    return y, rows.value


def conv_dgrad(dy, w, x_shape, stride, pad, add: Optional[torch.Tensor] = None):
    global launch_count
    N, Cin, H, W = x_shape
    Cout, _, R, S = w.shape
    dx = torch.empty(x_shape, dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
    check(lib.tmpi_conv_dgrad(dy.data_ptr(), w.data_ptr(), dx.data_ptr(), add.data_ptr() if add is not None else None,
                              N, H, W, Cin, Cout, R, S, stride, pad, stream_ptr()))
    launch_count += 1
    return dx


def conv_wgrad(dy, x, w_shape, stride, pad, out: Optional[torch.Tensor] = None, accumulate: bool = False):
    """``dW`` in the channels-last layout of the weight; ``out`` (a channels-last weight-shaped tensor, e.g. the
    parameter's gradient view) is written or accumulated in place when given."""
    global launch_count
    N, Cin, H, W = x.shape
    Cout, _, R, S = w_shape
    need = lib.tmpi_conv_wgrad_workspace_bytes(N, H, W, Cin, Cout, R, S, stride, pad)
    ws = _workspace(x.device, need)
    if out is None:
        out = torch.empty(w_shape, dtype=x.dtype, device=x.device).contiguous(memory_format=torch.channels_last)
        accumulate = False
    check(lib.tmpi_conv_wgrad(dy.data_ptr(), x.data_ptr(), out.data_ptr(), N, H, W, Cin, Cout, R, S, stride, pad,
                              ws.data_ptr(), ws.numel(), int(accumulate), stream_ptr()))
    launch_count += 2
    return out


def matmul_tn_splitk(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``a.T @ b`` for row-major ``a [K, M]`` and ``b [K, N]`` with a long ``K`` and a small output (a weight
    gradient over many rows): ``K`` is split over the SMs.  Rows of ``a`` / ``b`` may be pitched views."""
    global launch_count
    K, M = a.shape
    N = b.shape[1]
    ok = (has_symbol("tmpi_gemm_bf16_tn_splitk") and a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
          and M % 8 == 0 and N % 8 == 0 and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0
          and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)
    if not ok:
        r = torch.matmul(a.t(), b)
        if out is None:
            return r
        return out.add_(r) if accumulate else out.copy_(r)
    need = lib.tmpi_gemm_tn_splitk_workspace_bytes(M, N, K)
    ws = _workspace(a.device, need)
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
        accumulate = False
    check(lib.tmpi_gemm_bf16_tn_splitk(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                       ws.data_ptr(), ws.numel(), int(accumulate), stream_ptr()))
    launch_count += 2
    return out


def check_status() -> None:
    st = lib.tmpi_conv_status()
    if st:
        raise TorchMPIError(3, f"convolution kernel: a bounded wait ran out (code {st})")


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, stride, pad, stats, state=None):
        """``state`` (a dict, optional): receives ``rows`` (rows of partial sums written to ``stats``); may carry
        ``param`` (the Parameter behind ``w``: its gradient is then added into ``param.grad`` in place when a flat
        bucket owns that buffer) and ``fork`` (a ``GradFork`` shared by all consumers of ``x``)."""
        x, w = _cl(x), _cl(w)
        y, rows = conv_forward(x, w, stride, pad, stats)
        ctx.save_for_backward(x, w)
        ctx.stride, ctx.pad = stride, pad
        ctx.param = ctx.fork = None
        if state is not None:
            state["rows"] = rows
            ctx.param, ctx.fork = state.get("param"), state.get("fork")
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = _cl(dy)
        from ..parallel.flat_buckets import direct_grad, grad_written
        dx = dw = None
        if ctx.needs_input_grad[0]:
            def make_dx(add):
                if ctx.stride == 1:
                    return conv_dgrad(dy, w, x.shape, 1, ctx.pad, add=_cl(add) if add is not None else None)
                # strided input gradients stay on the library
                g = torch.ops.aten.convolution_backward(dy, x, w, None, (ctx.stride,) * 2, (ctx.pad,) * 2, (1, 1), False,
                                                        (0, 0), 1, (True, False, False))[0]
                return g if add is None else g.add_(add)
            dx = ctx.fork.offer(make_dx) if ctx.fork is not None else make_dx(None)
        if ctx.needs_input_grad[1]:
            sink = direct_grad(ctx.param)
            if sink is not None and sink.shape == w.shape and sink.stride() == w.stride() and sink.dtype == w.dtype:
                conv_wgrad(dy, x, w.shape, ctx.stride, ctx.pad, out=sink, accumulate=True)
                grad_written(ctx.param)
            else:
                dw = conv_wgrad(dy, x, w.shape, ctx.stride, ctx.pad)
        return dx, dw, None, None, None, None


def conv2d(x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0) -> torch.Tensor:
    if supported(x, w, stride, padding) and own_kernel_enabled(w.shape[2]):
        return _ConvFn.apply(x, w, stride, padding, None)
    return F.conv2d(x, w, None, stride, padding)


def conv_bn(conv: nn.Conv2d, bn, x: torch.Tensor, residual: Optional[torch.Tensor] = None, fork=None, res_fork=None) -> torch.Tensor:
    """``bn(conv(x), residual)`` for a ``FusedBatchNormReLU`` ``bn``.  In training, when both kernels apply, the
    convolution's epilogue accumulates the batch statistics of its output (per-CTA partial sums in the
    batch-norm's scratch buffer) and the batch-norm starts at its finalize step: the statistics pass over the
    activation, one full read of it, is gone.  ``fork`` / ``res_fork`` (``GradFork``, optional) are shared with the
    other consumers of ``x`` / of ``residual``: the gradients into those tensors are then summed inside the kernels."""
    from . import bn_relu
    w = conv.weight
    stride, pad = conv.stride[0], conv.padding[0]
    fused_bn = isinstance(bn, bn_relu.FusedBatchNormReLU)
    bn_kw = {"res_fork": res_fork} if (fused_bn and res_fork is not None) else {}
    if not supported(x, w, stride, pad) or not own_kernel_enabled(w.shape[2]):
        if fork is not None:
            fork.consumers -= 1       # a library convolution: autograd itself adds its gradient into x
        return bn(F.conv2d(x, w, None, conv.stride, conv.padding), residual, **bn_kw)
    fn_state = {"param": w, "fork": fork}
    fuse = (bn.training and x.dtype == torch.bfloat16 and bn.weight.dtype == torch.float32
            and has_symbol("tmpi_bn_relu_fwd_partials") and fused_bn)
    if not fuse:
        return bn(_ConvFn.apply(x, w, stride, pad, None, fn_state), residual, **bn_kw)
    stats = bn_relu._scratch_for(x.device, w.shape[0]).view(torch.float32)
    y = _ConvFn.apply(x, w, stride, pad, stats, fn_state)
    if not bn_relu.supported(y):
        return bn(y, residual, **bn_kw)
    return bn(y, residual, partial_rows=fn_state["rows"], **bn_kw)


def own_kernel_enabled(kernel_size: int) -> bool:
    """1x1 convolutions always run on the implicit-GEMM kernel; filters with taps only when ``conv_own_3x3`` is set."""
    from .. import config
    return kernel_size == 1 or bool(config.get("conv_own_3x3"))


class Conv2d(nn.Conv2d):
    """``nn.Conv2d`` (no bias, no groups, no dilation) whose three passes run on the implicit-GEMM kernel."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, padding: int = 0):
        super().__init__(in_channels, out_channels, kernel_size, stride=stride, padding=padding, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return conv2d(x, self.weight, self.stride[0], self.padding[0])
