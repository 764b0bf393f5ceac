"""Softmax cross-entropy whose forward also produces the gradient (one kernel, one read of the logits).

``cross_entropy(logits, labels)`` = mean over rows of ``logsumexp(x) - x[label]``.  On CUDA tensors the
forward kernel writes ``(softmax - onehot) / rows`` next to the loss, so backward is a scalar multiply.
The sum over rows is done by the last block in row order: the loss is bit-reproducible.
"""
from __future__ import annotations

import torch

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr

_scratch = {}
launch_count = 0     # kernels launched by this module (read by the benchmark)


def _scratch_for(dev: torch.device, rows: int) -> torch.Tensor:
    key = (dev.index, rows)
    if key not in _scratch:
        _scratch[key] = torch.zeros(lib.tmpi_xent_scratch_bytes(rows), dtype=torch.uint8, device=dev)
    return _scratch[key]


class _XentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, labels: torch.Tensor, unit_grad: bool = False):
        global launch_count
        ctx.unit_grad = unit_grad
        launch_count += 1
        rows, cols = logits.shape
        # rows may sit in a wider buffer (a [T, 50257] logit matrix kept with a pitch of 50264 so that the
        # GEMMs around it can use 16-byte rows): the kernel takes the pitch, and the gradient keeps it
        if logits.stride(1) == 1 and logits.stride(0) >= cols and rows > 1:
            x, ld = logits, logits.stride(0)
        else:
            x, ld = logits.contiguous(), cols
        buf = torch.empty((rows, ld), dtype=x.dtype, device=x.device)
        loss = torch.empty(1, dtype=torch.float32, device=x.device)
        check(lib.tmpi_xent_fwd_bwd_ld(x.data_ptr(), dtype_code(x.dtype), labels.data_ptr(), rows, cols, ld,
                                       loss.data_ptr(), buf.data_ptr(), 1.0 / rows,
                                       _scratch_for(x.device, rows).data_ptr(), stream_ptr()))
        ctx.grad_buf, ctx.cols = buf, cols
        return loss[0] / rows

    @staticmethod
    def backward(ctx, grad_out):
        buf, ctx.grad_buf = ctx.grad_buf, None          # scaled in place: backward runs once
        if not ctx.unit_grad:
            buf.mul_(grad_out.to(buf.dtype))
        return buf[:, :ctx.cols], None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, unit_grad: bool = False) -> torch.Tensor:
    """``unit_grad=True`` is a promise that backward starts at this loss (``loss.backward()``, incoming gradient
    1): the stored gradient is then handed on as it is, without a pass that multiplies it by the incoming
    gradient.  A scaled or combined loss must leave it off."""
    if logits.is_cuda:
        if not has_symbol("tmpi_xent_fwd_bwd"):
            raise RuntimeError("torchmpi_b200: native kernel 'tmpi_xent_fwd_bwd' is missing")
        if logits.dim() != 2 or labels.dtype != torch.int64:
            raise ValueError("cross_entropy expects [rows, classes] logits and int64 labels")
        return _XentFn.apply(logits, labels.contiguous(), unit_grad)
    return torch.nn.functional.cross_entropy(logits.float(), labels)


class CrossEntropyLoss(torch.nn.Module):
    def __init__(self, unit_grad: bool = False):
        super().__init__()
        self.unit_grad = unit_grad

    def forward(self, logits, labels):
        return cross_entropy(logits, labels, self.unit_grad)
