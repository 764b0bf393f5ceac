"""Tensor-parallel MLP benchmark: 4 layers (2 column/row blocks), d = 8192, hidden 32768, GELU, bf16.

    python -m torch.distributed.run --nproc-per-node 8 -m torchmpi_b200.parallel.bench_tp [--tokens 8192]

Each rank holds tokens/R rows of the input and 1/R of every weight.  Forward and backward run on the
fused all-gather->GEMM and GEMM->reduce-scatter kernels.  Reports, device-timed (CUDA events, max
over ranks, 3+ warm-up steps; the per-step working set of several GB exceeds the L2):
  * ms per forward+backward step and the TFLOP/s per GPU of the six GEMMs per block;
  * each fused kernel in isolation against its roofline = the slower of FLOPs / measured bf16 peak and
    NVLink bytes / link bandwidth;
  * ``--baseline``: the same block with NCCL all-gather / reduce-scatter around cuBLAS matmuls.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch
import torch.distributed as dist


def timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=8192)
    ap.add_argument("--d-hidden", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--n-comm", type=int, default=0, help="copy CTAs of ag_gemm (0: chosen from the tile count)")
    ap.add_argument("--baseline", action="store_true")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()

    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    from torchmpi_b200.parallel.tensor_parallel import TensorParallelMLP
    config.set("heap_bytes", 3 << 30)
    mpi.start(with_cuda=True)
    rank, R, dev = mpi.rank(), mpi.size(), mpi.device
    M, D, F = args.tokens, args.d_model, args.d_hidden
    rows, f = M // R, F // R
    peaks = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak_tf = json.loads(peaks.read_text())["bf16_tflops_sustained"] if peaks.exists() else 1400.0
    g = torch.Generator().manual_seed(7 + rank)
    x = torch.randn(rows, D, generator=g).to(dev).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(rows, D, generator=g).to(dev).to(torch.bfloat16)
    out = {"config": {"tokens": M, "d_model": D, "d_hidden": F, "layers": args.layers, "world": R,
                      "dtype": "bf16", "data": "synthetic N(0,1), random-init weights"}}

    if not args.baseline:
        model = TensorParallelMLP(rows, D, F, args.layers, bias=True, n_comm=args.n_comm)
        tp = model.tp

        def step():
            y = model(x)
            y.backward(dy)
        ms = timed(step, args.warmup, args.iters)
        tp.check()
        blocks = args.layers // 2
        flops = blocks * 6 * 2.0 * M * D * f               # per rank: 2 fwd + 4 bwd GEMMs per block
        out.update({"impl": "fused", "ms_per_step": ms, "tflops_per_gpu": flops / ms / 1e9,
                    "frac_of_sustained_peak": flops / ms / 1e9 / peak_tf})
        # the fused kernels alone
        blk = model[0]
        xs = x.detach()
        z = [None]
        ms_ag = timed(lambda: z.__setitem__(0, tp.ag_gemm(xs, blk.full_off, blk.full_buf, blk.w1, blk.b1)), 3, args.iters)
        h = torch.nn.functional.gelu(z[0])
        ms_rs = timed(lambda: tp.gemm_rs(h, blk.w2), 3, args.iters)
        gemm_flops = 2.0 * M * D * f
        link_bytes = (R - 1) / R * M * D * 2
        roof_ms = max(gemm_flops / (peak_tf * 1e9), link_bytes / (args.link_gbs * 1e6))
        out["ag_gemm"] = {"ms": ms_ag, "tflops": gemm_flops / ms_ag / 1e9, "roofline_ms": roof_ms,
                          "roofline_frac": roof_ms / ms_ag}
        out["gemm_rs"] = {"ms": ms_rs, "tflops": gemm_flops / ms_rs / 1e9, "roofline_ms": roof_ms,
                          "roofline_frac": roof_ms / ms_rs}
        tp.check()
    else:
        # NCCL + cuBLAS version of the same block
        import math
        w1 = [(torch.randn(f, D, device=dev) / math.sqrt(D)).to(torch.bfloat16).requires_grad_(True)
              for _ in range(args.layers // 2)]
        w2 = [(torch.randn(D, f, device=dev) / math.sqrt(F)).to(torch.bfloat16).requires_grad_(True)
              for _ in range(args.layers // 2)]
        b1 = [torch.zeros(f, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in w1]
        b2 = [torch.zeros(D, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in w1]

        class AG(torch.autograd.Function):
            @staticmethod
            def forward(ctx, t):
                full = torch.empty(M, t.shape[1], dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(full, t.contiguous())
                return full

            @staticmethod
            def backward(ctx, gfull):
                o = torch.empty(rows, gfull.shape[1], dtype=gfull.dtype, device=gfull.device)
                dist.reduce_scatter_tensor(o, gfull.contiguous())
                return o

        class RS(torch.autograd.Function):
            @staticmethod
            def forward(ctx, t):
                o = torch.empty(rows, t.shape[1], dtype=t.dtype, device=t.device)
                dist.reduce_scatter_tensor(o, t.contiguous())
                return o

            @staticmethod
            def backward(ctx, go):
                full = torch.empty(M, go.shape[1], dtype=go.dtype, device=go.device)
                dist.all_gather_into_tensor(full, go.contiguous())
                return full

        def step():
            h = x
            lin = torch.nn.functional.linear
            for a, ba, b, bb in zip(w1, b1, w2, b2):          # the same block: biases on both layers
                h = RS.apply(lin(torch.nn.functional.gelu(lin(AG.apply(h), a, ba)), b)) + bb
            h.backward(dy)
        ms = timed(step, args.warmup, args.iters)
        flops = (args.layers // 2) * 6 * 2.0 * M * D * f
        out.update({"impl": "nccl+cublas", "ms_per_step": ms, "tflops_per_gpu": flops / ms / 1e9,
                    "frac_of_sustained_peak": flops / ms / 1e9 / peak_tf})
    if rank == 0:
        print(json.dumps(out))
    mpi.stop()


if __name__ == "__main__":
    main()
