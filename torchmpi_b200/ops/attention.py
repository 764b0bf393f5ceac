"""Causal self-attention on the hand-written tcgen05 kernel (csrc/kernels/attention.cu).

``causal_attention(qkv, n_head)`` takes the output of a fused QKV projection, ``[B, T, 3 C]`` in bf16 with head size
64, and returns ``[B, T, C]``: the kernel reads Q, K and V where the projection left them (three tensor maps over
the same buffer) and writes the heads side by side, so there is no transpose before or after it.  It also returns
the row-wise log-sum-exp that a backward pass needs.

Forward and backward are this package's kernels (csrc/kernels/attention.cu, attention_bwd.cu).  ``_BACKWARDS`` can
put a library backward first instead, fed with this forward's output and log-sum-exp: cuDNN's attention backward (``aten._scaled_dot_product_cudnn_attention_backward``, 112 us for
8 x 16 x 1024 x 64 on a B200), else PyTorch's flash-attention backward (246 us); if neither operator accepts the
call, the backward recomputes the attention with ``F.scaled_dot_product_attention`` under autograd.
``last_backward`` says which one ran.  Shapes the kernel does
not take (head size other than 64, T not a multiple of 128, other dtypes, CPU) use
``F.scaled_dot_product_attention`` throughout.  The reference has no attention (its models are MNIST networks).
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F

from .._lib import lib, check, has_symbol, stream_ptr, TorchMPIError

launch_count = 0
last_backward = ""
HEAD = 64
# backward kernels in order of preference: this package's, then the libraries'; TORCHMPI_ATTENTION_BACKWARD=cudnn
# (or flash) puts a library first
_BACKWARDS = ("own", "cudnn", "flash")
_first = os.environ.get("TORCHMPI_ATTENTION_BACKWARD", "")
if _first in _BACKWARDS:
    _BACKWARDS = (_first,) + tuple(b for b in _BACKWARDS if b != _first)


def supported(qkv: torch.Tensor, n_head: int) -> bool:
    if not (has_symbol("tmpi_attention_fwd") and qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 3):
        return False
    B, T, C3 = qkv.shape
    return C3 == 3 * n_head * HEAD and T >= 128 and T % 128 == 0 and qkv.is_contiguous() and qkv.data_ptr() % 16 == 0


def check_status() -> None:
    """Raises if an attention CTA gave up on one of its bounded waits since the last call."""
    st = lib.tmpi_attention_status() or (lib.tmpi_attention_bwd_status() if has_symbol("tmpi_attention_bwd") else 0)
    if st:
        raise TorchMPIError(f"attention kernel: a bounded wait ran out (code {st})")


def attention_forward(qkv: torch.Tensor, n_head: int, need_lse: bool = True):
    """(out [B, T, C], lse [B, H, T] fp32 or None) of causal attention over the packed projection ``qkv``."""
    global launch_count
    B, T, C3 = qkv.shape
    C = C3 // 3
    out = torch.empty((B, T, C), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((B, n_head, T), dtype=torch.float32, device=qkv.device) if need_lse else None
    base, es = qkv.data_ptr(), qkv.element_size()
    check(lib.tmpi_attention_fwd(base, base + C * es, base + 2 * C * es, C3, out.data_ptr(), C,
                                 lse.data_ptr() if need_lse else None, B, T, n_head, 1.0 / math.sqrt(HEAD), stream_ptr()))
    launch_count += 1
    return out, lse


def attention_backward(qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor, n_head: int) -> torch.Tensor:
    """Gradient of the packed projection ``[B, T, 3 C]`` on this package's backward kernel: dK and dV are written
    into their column blocks by the main kernel, dQ is accumulated in fp32 and rounded into its block by a last pass."""
    global launch_count
    B, T, C3 = qkv.shape
    C = C3 // 3
    dout = dout.contiguous()
    dqkv = torch.empty_like(qkv)
    dq_acc = torch.empty((B * T, C), dtype=torch.float32, device=qkv.device)      # cleared by the kernel's first stage
    delta = torch.empty((B, n_head, T), dtype=torch.float32, device=qkv.device)
    base, gbase, es = qkv.data_ptr(), dqkv.data_ptr(), qkv.element_size()
    check(lib.tmpi_attention_bwd(base, base + C * es, base + 2 * C * es, C3, out.data_ptr(), C, dout.data_ptr(), C,
                                 lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), gbase, gbase + C * es, gbase + 2 * C * es,
                                 C3, B, T, n_head, 1.0 / math.sqrt(HEAD), stream_ptr()))
    launch_count += 1
    return dqkv


def _reference(qkv: torch.Tensor, n_head: int) -> torch.Tensor:
    B, T, C3 = qkv.shape
    C = C3 // 3
    q, k, v = (t.view(B, T, n_head, C // n_head).transpose(1, 2) for t in qkv.split(C, dim=2))
    return F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, n_head):
        out, lse = attention_forward(qkv, n_head)
        ctx.save_for_backward(qkv, out, lse)
        ctx.n_head = n_head
        return out

    @staticmethod
    def backward(ctx, dout):
        global last_backward
        qkv, out, lse = ctx.saved_tensors
        H = ctx.n_head
        B, T, C3 = qkv.shape
        C = C3 // 3
        heads = lambda t: t.view(B, T, H, HEAD).transpose(1, 2)          # [B, H, T, 64] views, nothing moves
        q, k, v = (heads(t) for t in qkv.split(C, dim=2))
        scale = 1.0 / math.sqrt(HEAD)
        zero = torch.zeros((), dtype=torch.int64, device=qkv.device)          # dropout state: unused at p = 0
        go, o = heads(dout.contiguous()), heads(out)
        grads = None
        for name in _BACKWARDS:
            if name == "own":              # this package's kernel: an error of it is raised, not routed around
                last_backward = name
                return attention_backward(qkv, out, lse, dout, H), None
            try:
                if name == "cudnn":
                    grads = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
                        go, q, k, v, o, lse.unsqueeze(-1), zero, zero, None, None, None, T, T, 0.0, True, scale=scale)
                elif name != "flash":
                    continue
                else:
                    grads = torch.ops.aten._scaled_dot_product_flash_attention_backward(
                        go, q, k, v, o, lse, None, None, T, T, 0.0, True, zero, zero, scale=scale)
                last_backward = name
                break
            except (RuntimeError, TypeError):
                continue
        if grads is None:
            with torch.enable_grad():
                leaf = qkv.detach().requires_grad_(True)
                (dqkv,) = torch.autograd.grad(_reference(leaf, H), leaf, dout)
            last_backward = "recompute"
            return dqkv, None
        dq, dk, dv = grads
        dqkv = torch.empty_like(qkv)
        for i, g in enumerate((dq, dk, dv)):
            dqkv[:, :, i * C:(i + 1) * C].view(B, T, H, HEAD).copy_(g.transpose(1, 2))
        return dqkv, None


def causal_attention(qkv: torch.Tensor, n_head: int) -> torch.Tensor:
    """Causal multi-head attention over a packed ``[B, T, 3 C]`` projection; returns ``[B, T, C]``."""
    if not supported(qkv, n_head):
        return _reference(qkv, n_head)
    return _AttnFn.apply(qkv, n_head)
