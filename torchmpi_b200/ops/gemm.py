"""bf16 GEMM on tcgen05 tensor cores (csrc/kernels/gemm_tcgen05.cu) and a Linear layer built on it.

``matmul_nt(a, b)`` computes ``a @ b.T`` for row-major ``a [M, K]`` and ``b [N, K]`` (K contiguous,
bf16), optionally with bias and GELU in the epilogue.  ``linear(x, w, bias, gelu)`` is the autograd
version: ``dX = dY @ W`` (``matmul_nn``) and ``dW = dY.T @ X`` (``matmul_tn``) read their operands as they
lie, through MN-major shared-memory descriptors, so backward makes no transposed copies.
"""
from __future__ import annotations

from typing import Optional

import torch

from .._lib import lib, check, dtype_code, has_symbol, stream_ptr, TorchMPIError

EPI_NONE, EPI_BIAS, EPI_GELU = 0, 1, 2
B_IS_KN = 4          # flag in the same word: the second operand is [K, N] with N contiguous
A_IS_KM = 8          # the first operand is [K, M] with M contiguous


def config_get(name: str) -> int:
    from .. import config
    return config.get(name)
launch_count = 0


def supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (a.is_cuda and b.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and
            a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1] and a.shape[1] % 8 == 0 and
            has_symbol("tmpi_gemm_bf16"))


def matmul_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(a @ b.T + bias)`` with fp32 accumulation; a: [M, K], b: [N, K], both bf16 and contiguous."""
    global launch_count
    if not has_symbol("tmpi_gemm_bf16"):
        raise RuntimeError("torchmpi_b200: native kernel 'tmpi_gemm_bf16' is missing")
    if not supported(a, b):
        raise ValueError("matmul_nt expects bf16 CUDA matrices [M, K] and [N, K] with K a multiple of 8")
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    epi = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if gelu else 0)
    check(lib.tmpi_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(),
                             bias.contiguous().data_ptr() if bias is not None else None, M, N, K, epi, stream_ptr()))
    launch_count += 1
    return out


def pair_kernel_takes(M: int, N: int, K: int) -> bool:
    """Shapes for which the CTA-pair kernel (and with it the ``[K, N]`` operand form) is available."""
    from .. import config
    return bool(config.get("gemm_pair")) and M >= 256 and N >= 256 and N % 8 == 0 and K % 8 == 0


def matmul_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a @ b`` for row-major ``a [M, K]`` and ``b [K, N]`` (N contiguous): the kernel reads ``b`` as it
    lies, through an MN-major shared-memory descriptor, where ``matmul_nt`` would need a transposed
    copy.  Shapes the CTA-pair kernel does not take fall back to that copy."""
    global launch_count
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape
    N = b.shape[1]
    if not (pair_kernel_takes(M, N, K) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda):
        return matmul_nt(a, b.t().contiguous(), out=out)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    check(lib.tmpi_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), None, M, N, K, B_IS_KN, stream_ptr()))
    launch_count += 1
    return out


def matmul_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a.T @ b`` for row-major ``a [K, M]`` and ``b [K, N]``: both operands are read as they lie
    (MN-major descriptors), which is the layout of a weight gradient ``dY.T @ X``.  Shapes the CTA-pair
    kernel does not take fall back to transposed copies."""
    global launch_count
    a, b = a.contiguous(), b.contiguous()
    K, M = a.shape
    N = b.shape[1]
    ok = (bool(config_get("gemm_pair")) and M >= 256 and N >= 256 and M % 8 == 0 and N % 8 == 0 and a.is_cuda
          and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16)
    if not ok:
        return matmul_nt(a.t().contiguous(), b.t().contiguous(), out=out)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    check(lib.tmpi_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), None, M, N, K, A_IS_KM | B_IS_KN, stream_ptr()))
    launch_count += 1
    return out


def check_status() -> None:
    """Raises if a GEMM CTA gave up on one of its bounded waits since the last call."""
    st = lib.tmpi_gemm_status()
    if st:
        raise TorchMPIError(3, f"tcgen05 GEMM: a bounded wait ran out (code {st})")


def _gemm_ex(a, b, c, M, N, K, lda, ldb, ldc, flags):
    global launch_count
    check(lib.tmpi_gemm_bf16_ex(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, M, N, K, lda, ldb, ldc, flags, stream_ptr()))
    launch_count += 1


class _WideHeadFn(torch.autograd.Function):
    """``x @ w.T`` for an output width that is not a multiple of 8 (a vocabulary of 50257).  A library GEMM
    falls back to unvectorised kernels for such a matrix; here the result lives in a buffer whose row pitch
    is rounded up to 8 elements and a view of its first ``V`` columns is returned, so that all three GEMMs
    (forward, dX, dW) run on the CTA-pair kernel with explicit pitches and no padding copies."""

    @staticmethod
    def forward(ctx, x2, w):
        T, d = x2.shape
        V = w.shape[0]
        Vp = (V + 7) // 8 * 8
        buf = torch.empty((T, Vp), dtype=x2.dtype, device=x2.device)
        _gemm_ex(x2, w, buf, T, V, d, d, d, Vp, 0)
        ctx.save_for_backward(x2, w)
        return buf[:, :V]

    @staticmethod
    def backward(ctx, dl):
        x2, w = ctx.saved_tensors
        T, d = x2.shape
        V = w.shape[0]
        if not (dl.stride(1) == 1 and dl.stride(0) % 8 == 0 and dl.data_ptr() % 16 == 0):
            pad = torch.zeros((T, (V + 7) // 8 * 8), dtype=dl.dtype, device=dl.device)
            pad[:, :V] = dl
            dl = pad[:, :V]
        ld = dl.stride(0)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty((T, d), dtype=x2.dtype, device=x2.device)
            _gemm_ex(dl, w, dx, T, d, V, ld, d, d, B_IS_KN)                  # dX = dL @ W, W read as [K = V, N = d]
        if ctx.needs_input_grad[1]:
            dw = torch.empty((V, d), dtype=w.dtype, device=w.device)
            _gemm_ex(dl, x2, dw, V, d, T, ld, d, d, A_IS_KM | B_IS_KN)       # dW = dL.T @ X, both as stored
        return dx, dw


def wide_head(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x2 @ w.T`` (``x2 [T, d]``, ``w [V, d]``) for any ``V``; see ``_WideHeadFn``.  Falls back to
    ``F.linear`` when the CTA-pair kernel does not apply."""
    T, d = x2.shape
    V = w.shape[0]
    if (x2.is_cuda and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and T >= 256 and V >= 256 and d >= 256
            and d % 8 == 0 and T % 8 == 0 and bool(config_get("gemm_pair")) and has_symbol("tmpi_gemm_bf16_ex")
            and x2.is_contiguous() and w.is_contiguous()):
        return _WideHeadFn.apply(x2, w)
    return torch.nn.functional.linear(x2, w)


def gelu(z: torch.Tensor) -> torch.Tensor:
    """``gelu(z)`` (erf form, no autograd) through ``tmpi_gelu_fwd`` (csrc/kernels/bias_grad.cu: rational erf, so the pass
    is memory bound) where it applies; ``F.gelu`` otherwise.  ``bias_grad(dy, z)`` is its backward."""
    global launch_count
    if not (z.is_cuda and z.is_contiguous() and z.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and (z.numel() * z.element_size()) % 16 == 0 and z.data_ptr() % 16 == 0 and has_symbol("tmpi_gelu_fwd")):
        return torch.nn.functional.gelu(z)
    y = torch.empty_like(z)
    st = lib.tmpi_gelu_fwd(z.data_ptr(), y.data_ptr(), z.numel(), dtype_code(z.dtype), stream_ptr())
    if st:
        check(st)
    launch_count += 1
    return y


_gelu_kernel = gelu          # `_LinearFn.forward` has a flag named `gelu`
_bg_scratch = {}
_bg_need = {}


def bias_grad(dy2: torch.Tensor, z: Optional[torch.Tensor] = None):
    """``(dz, db)`` with ``dz = dy2 * gelu'(z)`` (``dy2`` itself when ``z`` is None) and ``db = dz.sum(0)``, in one
    pass over ``dy2`` (and ``z``) where the kernel applies (csrc/kernels/bias_grad.cu); PyTorch ops otherwise."""
    global launch_count
    rows, C = dy2.shape
    per_slab = 128 * (16 // dy2.element_size())
    if not (dy2.is_cuda and dy2.is_contiguous() and C % per_slab == 0 and has_symbol("tmpi_bias_grad")
            and dy2.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and (z is None or (z.is_contiguous() and z.dtype == dy2.dtype))):
        dz = torch.ops.aten.gelu_backward(dy2, z) if z is not None else dy2
        return dz, dz.sum(0)
    sp = stream_ptr()
    key = (dy2.device.index, sp)
    need = _bg_need.get(C)
    if need is None:
        need = _bg_need[C] = lib.tmpi_bias_grad_scratch_bytes(C)
    buf = _bg_scratch.get(key)
    if buf is None or buf.numel() < need:
        buf = _bg_scratch[key] = torch.empty(need, dtype=torch.uint8, device=dy2.device)
    db = torch.empty(C, dtype=dy2.dtype, device=dy2.device)
    if z is None:
        dz = dy2
        st = lib.tmpi_bias_grad(dy2.data_ptr(), None, None, db.data_ptr(), rows, C, dtype_code(dy2.dtype), buf.data_ptr(), sp)
    else:
        dz = torch.empty_like(dy2)
        st = lib.tmpi_bias_grad(dy2.data_ptr(), z.data_ptr(), dz.data_ptr(), db.data_ptr(), rows, C, dtype_code(dy2.dtype),
                                buf.data_ptr(), sp)
    if st:
        check(st)
    launch_count += 2
    return dz, db


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, gelu):
        x2 = x.reshape(-1, x.shape[-1])
        if gelu:
            z = matmul_nt(x2, w, bias)                       # pre-activation is needed by backward
            y = _gelu_kernel(z)
            ctx.save_for_backward(x2, w, z)
        else:
            y = matmul_nt(x2, w, bias)
            ctx.save_for_backward(x2, w, None)
        ctx.has_bias, ctx.gelu, ctx.shape = bias is not None, gelu, x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, z = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dy2, db = bias_grad(dy2, z if ctx.gelu else None)       # GELU backward and the column sum in one pass
        elif ctx.gelu:
            dy2 = torch.ops.aten.gelu_backward(dy2, z)
        dx = matmul_nn(dy2, w) if ctx.needs_input_grad[0] else None
        dw = matmul_tn(dy2, x2) if ctx.needs_input_grad[1] else None
        return (dx.reshape(ctx.shape) if dx is not None else None), dw, db, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False) -> torch.Tensor:
    """``gelu?(x @ w.T + bias)`` through the tcgen05 kernel when the operands qualify, else PyTorch."""
    rows = x.numel() // max(1, x.shape[-1])
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and w.shape[0] % 8 == 0 and rows % 8 == 0 and has_symbol("tmpi_gemm_bf16"):
        return _LinearFn.apply(x, w, bias, gelu)
    y = torch.nn.functional.linear(x, w, bias)
    return torch.nn.functional.gelu(y) if gelu else y


class Linear(torch.nn.Linear):
    """``nn.Linear`` whose matrix products run on the hand-written tcgen05 kernel."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gelu: bool = False, **kw):
        super().__init__(in_features, out_features, bias=bias, **kw)
        self.gelu = gelu

    def forward(self, x):
        return linear(x, self.weight, self.bias, self.gelu)
