"""Fused BatchNorm2d (+ residual add) (+ ReLU) for channels-last activations (csrc/kernels/bn_relu.cu).

``FusedBatchNormReLU(C, relu=True)`` is a drop-in for ``BatchNorm2d`` followed by an optional residual
add and ReLU: ``y = relu(bn(x) + residual)``.  Parameters and running statistics are fp32; activations
may be bf16 / fp16 / fp32.  Training forward is three launches (statistics, finalize, apply), backward
three more; eager PyTorch needs separate batch-norm, add and ReLU kernels each way.  CPU tensors and
channel counts the kernel does not cover take the PyTorch ops.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import config
from .._lib import lib, check, dtype_code, has_symbol, stream_ptr

launch_count = 0
_scratch = {}


def _scratch_for(dev: torch.device, C: int) -> torch.Tensor:
    key = (dev.index, stream_ptr())
    need = lib.tmpi_bn_scratch_bytes(C)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < need:
        buf = _scratch[key] = torch.empty(max(need, lib.tmpi_bn_scratch_bytes(2048)), dtype=torch.uint8, device=dev)
    return buf


def supported(x: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dim() == 4 and has_symbol("tmpi_bn_relu_fwd")):
        return False
    if x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return False
    V = 16 // x.element_size()
    C = x.shape[1]
    return C % V == 0 and 256 % (C // V) == 0


class _BnReluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, beta, running_mean, running_var, eps, momentum, relu, training, partial_rows=0,
                params=None, res_fork=None):
        """``partial_rows > 0``: the producer of ``x`` (a convolution of ``ops.conv``) has already left that many
        rows of partial sums in this stream's scratch buffer, so the statistics pass is skipped.  ``params``: the
        (weight, bias) Parameters, whose gradients are added in place when a flat bucket owns their buffers;
        ``res_fork``: a ``GradFork`` shared by the consumers of ``residual``."""
        global launch_count
        x = x.contiguous(memory_format=torch.channels_last)
        if residual is not None:
            residual = residual.contiguous(memory_format=torch.channels_last)
        N, C, H, W = x.shape
        rows = N * H * W
        y = torch.empty_like(x, memory_format=torch.channels_last)
        if training:
            mean = torch.empty(C, dtype=torch.float32, device=x.device)
            invstd = torch.empty(C, dtype=torch.float32, device=x.device)
        else:
            mean = running_mean.float()
            invstd = torch.rsqrt(running_var.float() + eps)
        # a ReLU layer with a residual keeps one mask bit per element for its backward (a sixteenth of y)
        bits = None
        if relu and residual is not None and any(ctx.needs_input_grad):
            bits = torch.empty(rows * C // (16 // x.element_size()), dtype=torch.uint8, device=x.device)
        if training and partial_rows > 0:
            check(lib.tmpi_bn_relu_fwd_partials(
                x.data_ptr(), residual.data_ptr() if residual is not None else None, y.data_ptr(),
                gamma.data_ptr(), beta.data_ptr(),
                running_mean.data_ptr() if running_mean is not None else None,
                running_var.data_ptr() if running_var is not None else None,
                mean.data_ptr(), invstd.data_ptr(), rows, C, eps, momentum, int(relu),
                dtype_code(x.dtype), bits.data_ptr() if bits is not None else None,
                _scratch_for(x.device, C).data_ptr(), int(partial_rows), stream_ptr()))
            launch_count += 2
        else:
            check(lib.tmpi_bn_relu_fwd(
                x.data_ptr(), residual.data_ptr() if residual is not None else None, y.data_ptr(),
                gamma.data_ptr(), beta.data_ptr(),
                running_mean.data_ptr() if (training and running_mean is not None) else None,
                running_var.data_ptr() if (training and running_var is not None) else None,
                mean.data_ptr(), invstd.data_ptr(), rows, C, eps, momentum, int(relu), int(training),
                dtype_code(x.dtype), bits.data_ptr() if bits is not None else None,
                _scratch_for(x.device, C).data_ptr(), stream_ptr()))
            launch_count += 3 if training else 1
        # a ReLU layer without a residual rebuilds its mask from x in backward; neither kind reads y again
        ctx.mask_from_x = relu and residual is None
        keep_y = relu and not ctx.mask_from_x and bits is None
        ctx.save_for_backward(x, y if keep_y else None, gamma, beta, mean, invstd, bits)
        ctx.relu, ctx.has_res = relu, residual is not None
        ctx.params, ctx.res_fork = params, res_fork
        return y

    @staticmethod
    def backward(ctx, dy):
        global launch_count
        x, y, gamma, beta, mean, invstd, bits = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        N, C, H, W = x.shape
        dx = torch.empty_like(x, memory_format=torch.channels_last)
        dres = torch.empty_like(x, memory_format=torch.channels_last) if ctx.has_res else None
        dgamma = torch.empty(C, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(C, dtype=torch.float32, device=x.device)
        from ..parallel.flat_buckets import direct_grad, grad_written
        acc_g = acc_b = None
        if ctx.params is not None and has_symbol("tmpi_bn_relu_bwd_acc"):
            acc_g, acc_b = direct_grad(ctx.params[0]), direct_grad(ctx.params[1])
            if acc_g is None or acc_b is None or not (acc_g.is_contiguous() and acc_b.is_contiguous()
                                                      and acc_g.dtype == torch.float32 and acc_b.dtype == torch.float32):
                acc_g = acc_b = None
        check(lib.tmpi_bn_relu_bwd_acc(
            x.data_ptr(), y.data_ptr() if y is not None else None, dy.data_ptr(), dx.data_ptr(),
            dres.data_ptr() if dres is not None else None, gamma.data_ptr(), beta.data_ptr(), mean.data_ptr(), invstd.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
            N * H * W, C, int(ctx.relu), dtype_code(x.dtype), bits.data_ptr() if bits is not None else None,
            _scratch_for(x.device, C).data_ptr(), acc_g.data_ptr() if acc_g is not None else None,
            acc_b.data_ptr() if acc_b is not None else None, stream_ptr()))
        launch_count += 3
        if acc_g is not None:                  # the parameter gradients were added in place by the finalize kernel
            grad_written(ctx.params[0])
            grad_written(ctx.params[1])
            dgamma = dbeta = None
        if dres is not None and ctx.res_fork is not None:
            dres = ctx.res_fork.offer(lambda add: dres if add is None else dres.add_(add))
        return dx, dres, dgamma, dbeta, None, None, None, None, None, None, None, None, None


class _BnReluPoolFn(torch.autograd.Function):
    """``max_pool2d(relu(batch_norm(x)), 3, 2, 1)`` without materialising the full-resolution activation."""

    @staticmethod
    def forward(ctx, x, gamma, beta, running_mean, running_var, eps, momentum, training):
        global launch_count
        x = x.contiguous(memory_format=torch.channels_last)
        N, C, H, W = x.shape
        OH, OW = (H - 1) // 2 + 1, (W - 1) // 2 + 1
        y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((N, OH, OW, C), dtype=torch.uint8, device=x.device)
        if training:
            mean = torch.empty(C, dtype=torch.float32, device=x.device)
            invstd = torch.empty(C, dtype=torch.float32, device=x.device)
        else:
            mean = running_mean.float()
            invstd = torch.rsqrt(running_var.float() + eps)
        check(lib.tmpi_bn_relu_pool_fwd(
            x.data_ptr(), y.data_ptr(), idx.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
            running_mean.data_ptr() if (training and running_mean is not None) else None,
            running_var.data_ptr() if (training and running_var is not None) else None,
            mean.data_ptr(), invstd.data_ptr(), N, H, W, C, eps, momentum, int(training), dtype_code(x.dtype),
            _scratch_for(x.device, C).data_ptr(), stream_ptr()))
        launch_count += 3 if training else 1
        ctx.save_for_backward(x, idx, gamma, beta, mean, invstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        global launch_count
        x, idx, gamma, beta, mean, invstd = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        N, C, H, W = x.shape
        dx = torch.empty_like(x, memory_format=torch.channels_last)
        dgamma = torch.empty(C, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(C, dtype=torch.float32, device=x.device)
        if config.get("bn_pool_fused_bwd"):
            # one stage: both batch-norm passes rebuild the pool's gradient routing from dy and the index
            check(lib.tmpi_bn_relu_pool_bwd(
                x.data_ptr(), dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                mean.data_ptr(), invstd.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), N, H, W, C, dtype_code(x.dtype),
                _scratch_for(x.device, C).data_ptr(), stream_ptr()))
            launch_count += 3
        else:
            # measured faster: route the gradient through the pool once, then the batch-norm backward with the
            # ReLU mask rebuilt from x (the rectified activation itself was never stored)
            OH, OW = dy.shape[2], dy.shape[3]
            da = torch.empty_like(x, memory_format=torch.channels_last)
            check(lib.tmpi_maxpool_bwd(dy.data_ptr(), idx.data_ptr(), da.data_ptr(), N, H, W, C, OH, OW, 3, 2, 1,
                                       dtype_code(x.dtype), stream_ptr()))
            check(lib.tmpi_bn_relu_bwd(
                x.data_ptr(), None, da.data_ptr(), dx.data_ptr(), None, gamma.data_ptr(), beta.data_ptr(),
                mean.data_ptr(), invstd.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), N * H * W, C, 1,
                dtype_code(x.dtype), None, _scratch_for(x.device, C).data_ptr(), stream_ptr()))
            launch_count += 4
        return dx, dgamma, dbeta, None, None, None, None, None


class FusedBatchNormReLUMaxPool(nn.BatchNorm2d):
    """``BatchNorm2d`` + ReLU + ``MaxPool2d(3, stride=2, padding=1)`` as one stage (the ResNet stem).  The
    parameters and buffers are those of the ``BatchNorm2d``."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__(num_features, eps=eps, momentum=momentum)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if supported(x) and self.weight.dtype == torch.float32 and has_symbol("tmpi_bn_relu_pool_fwd"):
            return _BnReluPoolFn.apply(x, self.weight, self.bias, self.running_mean, self.running_var, self.eps,
                                       self.momentum, self.training)
        out = torch.relu(F.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training,
                                      self.momentum, self.eps))
        return F.max_pool2d(out, 3, 2, 1)


class FusedBatchNormReLU(nn.BatchNorm2d):
    """``forward(x, residual=None)`` = ``relu(batch_norm(x) + residual)`` (ReLU optional)."""

    def __init__(self, num_features: int, relu: bool = True, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__(num_features, eps=eps, momentum=momentum)
        self.relu = relu

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, partial_rows: int = 0, res_fork=None) -> torch.Tensor:
        if supported(x) and self.weight.dtype == torch.float32:
            # num_batches_tracked is only needed for momentum=None (cumulative average), not supported here
            return _BnReluFn.apply(x, residual, self.weight, self.bias, self.running_mean, self.running_var,
                                   self.eps, self.momentum, self.relu, self.training, partial_rows,
                                   (self.weight, self.bias), res_fork)
        if res_fork is not None:
            res_fork.consumers -= 1            # the library path lets autograd add this gradient
        out = F.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training,
                           self.momentum, self.eps)
        if residual is not None:
            out = out + residual
        return torch.relu(out) if self.relu else out
