"""Tensor-parallel MLP blocks on the fused all-gather->GEMM and GEMM->reduce-scatter kernels.

The reference's model-parallel example (``nn.MPLinear``, examples/mnist/mnist_modelparallel.lua:30-60)
splits a Linear layer's input features over the ranks and allreduces outputs and input gradients.
Here a block is the usual column-split / row-split pair with the activations sharded by rows
(tokens) between blocks:

    x_shard [M/R, D] --all-gather--> X [M, D]
    Z = X W1_r^T + b1_r          (W1_r: this rank's [F/R, D] rows of the first weight)     ag_gemm
    H = gelu(Z)
    y_shard = reduce_scatter(H W2_r^T) + b2      (W2_r: this rank's [D, F/R] columns)        gemm_rs

Backward mirrors it: dY is all-gathered inside the GEMM that produces dH, and dX is reduce-scattered
by the GEMM that produces it; the two weight gradients are local GEMMs on the gathered operands.
All matrix products run on the tcgen05 kernel; every collective is fused into its GEMM
(csrc/kernels/gemm_fused.cu).  ``BlockSequential.tensor_parallel(...)`` builds a stack of such blocks.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import torch
import torch.nn as nn

from .. import _lib, runtime
from .._lib import lib, check, stream_ptr
from ..ops import gemm
from ..runtime import S


def _fn(name, res, args):
    f = getattr(lib, name)
    f.restype, f.argtypes = res, args
    return f


_i, _sz, _vp = C.c_int, C.c_size_t, C.c_void_p
_gp = C.POINTER(_lib.Group)
_ag_gemm = _fn("tmpi_cuda_ag_gemm", _i, [_sz, _sz, _vp, _vp, _vp, _i, _i, _i, _i, _i, _gp, _vp]) \
    if _lib.has_symbol("tmpi_cuda_ag_gemm") else None
_gemm_rs = _fn("tmpi_cuda_gemm_rs", _i, [_vp, _vp, _sz, _vp, _i, _i, _i, _i, _gp, _vp]) \
    if _lib.has_symbol("tmpi_cuda_gemm_rs") else None
_fused_status = _fn("tmpi_cuda_fused_gemm_status", _i, []) if _lib.has_symbol("tmpi_cuda_fused_gemm_status") else None

launch_count = 0


class TPGroup:
    """The ranks a tensor-parallel block spans, with the symmetric buffers its kernels need."""

    def __init__(self, rows_per_rank: int, d_model: int, members: Optional[Sequence[int]] = None, n_comm: int = 0):
        if S.cuda_heap is None or _ag_gemm is None:
            raise RuntimeError("tensor parallelism needs the CUDA symmetric heap and the fused GEMM kernels")
        self.heap = S.cuda_heap
        self.members = tuple(members) if members is not None else runtime.intra_members(runtime.collective_span()[0])
        self.R = len(self.members)
        self.me = self.members.index(S.rank)
        self.rows, self.d, self.n_comm = rows_per_rank, d_model, n_comm
        self.M = rows_per_rank * self.R
        bf = torch.bfloat16
        self.shard_buf, self.shard_off = self._alloc(rows_per_rank * d_model)      # staging of a row shard
        self.dfull_buf, self.dfull_off = self._alloc(self.M * d_model)             # gathered gradient
        self.slots_buf, self.slots_off = self._alloc(self.M * d_model)             # [R, rows, D] partial outputs
        self._arr = _lib.int_array(self.members)
        self._group = _lib.Group(self._arr, self.R, self.me, 0)
        del bf

    def _alloc(self, numel: int):
        raw, off = self.heap.alloc(numel * 2)
        return raw.view(torch.bfloat16), off

    def new_full_buffer(self):
        """A gathered-activation buffer [M, D] that a block keeps for its backward pass."""
        return self._alloc(self.M * self.d)

    def takes_kn(self) -> bool:
        """Whether the fused kernels accept the weight as ``[K, N]`` (the CTA-pair kernels do)."""
        from .. import config
        return bool(config.get("gemm_pair")) and self.rows % 256 == 0

    def ag_gemm(self, shard: torch.Tensor, full_off: int, full_buf: torch.Tensor, w: torch.Tensor,
                bias: Optional[torch.Tensor], gelu: bool = False, w_is_kn: bool = False) -> torch.Tensor:
        """``act(all_gather(shard) @ w.T + bias)``; the gathered operand is left in ``full_buf``.
        ``w_is_kn``: ``w`` is ``[K, N]`` and the product is ``all_gather(shard) @ w``."""
        global launch_count
        self.shard_buf[:shard.numel()].copy_(shard.reshape(-1))
        if w_is_kn and not self.takes_kn():
            w, w_is_kn = w.t().contiguous(), False
        K, N = w.shape if w_is_kn else (w.shape[1], w.shape[0])
        out = torch.empty((self.M, N), dtype=torch.bfloat16, device=shard.device)
        epi = (1 if bias is not None else 0) | (2 if gelu else 0) | (4 if w_is_kn else 0)
        check(_ag_gemm(self.shard_off, full_off, w.data_ptr(), out.data_ptr(),
                       bias.data_ptr() if bias is not None else None, self.M, N, K, epi, self.n_comm,
                       C.byref(self._group), stream_ptr()))
        launch_count += 1
        return out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, w_is_kn: bool = False) -> torch.Tensor:
        """``reduce_scatter_rows(a @ w.T)``: this rank's [rows, N] slice of the sum over ranks
        (``a @ w`` for a ``[K, N]`` weight with ``w_is_kn``)."""
        global launch_count
        if w_is_kn and not self.takes_kn():
            w, w_is_kn = w.t().contiguous(), False
        K, N = w.shape if w_is_kn else (w.shape[1], w.shape[0])
        assert N == self.d, "gemm_rs output width must be the model width the slot buffer was sized for"
        out = torch.empty((self.rows, N), dtype=torch.bfloat16, device=a.device)
        check(_gemm_rs(a.data_ptr(), w.data_ptr(), self.slots_off, out.data_ptr(), self.M, N, K,
                       4 if w_is_kn else 0, C.byref(self._group), stream_ptr()))
        launch_count += 1
        return out

    def check(self) -> None:
        st = _fused_status() if _fused_status else 0
        if st:
            raise _lib.TorchMPIError(3, f"fused GEMM: a bounded wait ran out (code {st})")
        self.heap.check_status(0)
        gemm.check_status()


class _TPMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w1, b1, w2, b2, tp: TPGroup, full_buf, full_off):
        z = tp.ag_gemm(x_shard, full_off, full_buf, w1, b1)           # [M, F/R] pre-activation
        h = gemm.gelu(z)
        y = tp.gemm_rs(h, w2)                                          # [rows, D]
        if b2 is not None:
            y = y + b2
        ctx.save_for_backward(w1, w2, z, h)
        ctx.tp, ctx.full_buf, ctx.has_b1, ctx.has_b2 = tp, full_buf, b1 is not None, b2 is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        w1, w2, z, h = ctx.saved_tensors
        tp: TPGroup = ctx.tp
        x_full = ctx.full_buf[:tp.M * tp.d].view(tp.M, tp.d)
        dy_shard = dy_shard.contiguous()
        dh = tp.ag_gemm(dy_shard, tp.dfull_off, tp.dfull_buf, w2, None, w_is_kn=True)        # [M, F/R] = dy @ w2
        dy_full = tp.dfull_buf[:tp.M * tp.d].view(tp.M, tp.d)
        # the two weight gradients are local GEMMs whose contraction dimension is the slow one of both
        # operands: the CTA-pair kernel reads them as they lie (MN-major descriptors)
        dw2 = gemm.matmul_tn(dy_full, h)                                                      # [D, F/R]
        db2 = gemm.bias_grad(dy_full)[1] if ctx.has_b2 else None
        dz, db1 = gemm.bias_grad(dh, z) if ctx.has_b1 else (torch.ops.aten.gelu_backward(dh, z), None)
        dx = tp.gemm_rs(dz, w1, w_is_kn=True)                                                 # [rows, D] = dz @ w1
        dw1 = gemm.matmul_tn(dz, x_full)                                                      # [F/R, D]
        return dx, dw1, db1, dw2, db2, None, None, None


class TensorParallelMLPBlock(nn.Module):
    """One column-split + row-split pair.  Input and output are row shards ``[M/R, D]``."""

    def __init__(self, tp: TPGroup, d_model: int, d_hidden: int, bias: bool = True, device=None):
        super().__init__()
        assert d_hidden % tp.R == 0
        self.tp = tp
        f = d_hidden // tp.R
        dev = device or S.device
        self.w1 = nn.Parameter(torch.empty(f, d_model, dtype=torch.bfloat16, device=dev))
        self.w2 = nn.Parameter(torch.empty(d_model, f, dtype=torch.bfloat16, device=dev))
        self.b1 = nn.Parameter(torch.zeros(f, dtype=torch.bfloat16, device=dev)) if bias else None
        self.b2 = nn.Parameter(torch.zeros(d_model, dtype=torch.bfloat16, device=dev)) if bias else None
        # slice r of the unsharded matrices is drawn from seed base + r: every rank can rebuild any slice
        g = torch.Generator(device="cpu").manual_seed(self.slice_seed(tp.me, d_hidden))
        with torch.no_grad():
            self.w1.copy_(torch.randn(f, d_model, generator=g) / math.sqrt(d_model))
            self.w2.copy_(torch.randn(d_model, f, generator=g) / math.sqrt(d_hidden))
        self.full_buf, self.full_off = tp.new_full_buffer()

    @staticmethod
    def slice_seed(rank: int, d_hidden: int) -> int:
        return 1234 + 7919 * rank + d_hidden

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _TPMLPFn.apply(x_shard, self.w1, self.b1, self.w2, self.b2, self.tp, self.full_buf, self.full_off)


class TensorParallelMLP(nn.Sequential):
    """``layers`` linear layers alternating column / row splits (= layers / 2 blocks) of width ``d_model`` and
    hidden width ``d_hidden``; activations travel between blocks as row shards."""

    def __init__(self, rows_per_rank: int, d_model: int = 8192, d_hidden: int = 32768, layers: int = 4,
                 bias: bool = True, members: Optional[Sequence[int]] = None, n_comm: int = 0):
        assert layers % 2 == 0
        tp = TPGroup(rows_per_rank, d_model, members, n_comm)
        super().__init__(*[TensorParallelMLPBlock(tp, d_model, d_hidden, bias) for _ in range(layers // 2)])
        self.tp = tp
