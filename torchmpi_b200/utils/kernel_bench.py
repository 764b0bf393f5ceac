"""Times the single-GPU hot kernels in isolation and reports them against the measured HBM peak.

``python -m torchmpi_b200.utils.kernel_bench [--kernel NAME] [--reps N] [--small]``

Each kernel runs on inputs larger than the 126 MB L2 (``--small`` keeps them just above it, for
profiler captures), after 3 warm-up launches, timed with CUDA events on the launching stream with a
synchronize on both sides; an L2-sized buffer is rewritten between timed launches.  Output: one JSON
line per kernel with the algorithmic bytes, the time, GB/s and the fraction of the copy bandwidth in
MEASURED_PEAKS.json (fallback 6650 GB/s when the file is absent).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def peak_gbs() -> tuple:
    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if f.exists():
        return json.loads(f.read_text())["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def time_kernel(fn, reps: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        flush.add_(1)                      # rewrite > L2 bytes so the next launch starts cold
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        # keep the GPU busy for ~0.4 ms while the host enqueues the events and the call, so that the interval is
        # the kernel's time on the device and not the host's launch path (descriptor encoding, Python, allocation)
        torch.cuda._sleep(800_000)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def cases(small: bool):
    from torchmpi_b200.ops import elementwise, xent, stats
    from torchmpi_b200.ops.bn_relu import _BnReluFn
    from torchmpi_b200._lib import lib, dtype_code, stream_ptr, check
    dev = torch.device("cuda")
    out = {}

    n = (40 if small else 128) << 20
    w = torch.randn(n, device=dev).to(torch.bfloat16)
    g = torch.randn(n, device=dev).to(torch.bfloat16)
    master, mom = w.float(), torch.zeros(n, device=dev)
    out["sgd_momentum_bf16_master"] = (
        lambda: elementwise.sgd_momentum_(w, g, lr=0.1, momentum=0.9, master=master, momentum_buf=mom, zero_grad=True),
        n * (2 + 4 + 4 + 4 + 4 + 2 + 2))   # grad r, master r/w, momentum r/w, weight w, grad zero w

    N, C, H = (64, 64, 112) if small else (256, 64, 112)
    x = torch.randn(N, C, H, H, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    res = torch.randn_like(x)
    gamma, beta = torch.ones(C, device=dev), torch.zeros(C, device=dev)
    rm, rv = torch.zeros(C, device=dev), torch.ones(C, device=dev)
    nb = x.numel() * 2

    def bn_fwd():
        return _BnReluFn.apply(x, res, gamma, beta, rm, rv, 1e-5, 0.1, True, True)
    out["bn_relu_add_fwd"] = (bn_fwd, nb * 4)          # x twice, residual once, y once

    xg = x.clone().requires_grad_(True)
    rg = res.clone().requires_grad_(True)
    y = _BnReluFn.apply(xg, rg, gamma.requires_grad_(True), beta.requires_grad_(True), rm, rv, 1e-5, 0.1, True, True)
    dy = torch.randn_like(y)

    def bn_bwd():
        torch.autograd.grad(y, (xg, rg), dy, retain_graph=True)
    out["bn_relu_add_bwd"] = (bn_bwd, nb * 8)          # (x, y, dy) twice, dx, dresidual

    rows, cols = (8192, 50257) if not small else (2048, 50257)
    logits = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
    labels = torch.randint(0, cols, (rows,), device=dev)
    out["xent_fwd_bwd"] = (lambda: xent._XentFn.apply(logits, labels), rows * cols * 2 * 2)  # x once (the row is kept in shared memory), dx once

    big = torch.randn((64 if small else 256) << 20, device=dev)
    stat_scratch = torch.zeros(lib.tmpi_absmean_var_scratch_bytes(), dtype=torch.uint8, device=dev)
    stat_out = torch.empty(2, dtype=torch.float64, device=dev)

    def absstat():                  # the kernel alone (stats.absmean_var adds a device-to-host read of the two sums)
        check(lib.tmpi_absmean_var(big.data_ptr(), dtype_code(big.dtype), big.numel(), stat_out.data_ptr(),
                                   stat_scratch.data_ptr(), stream_ptr()))
    out["absmean_var"] = (absstat, big.numel() * 4)
    out["absmean_var_with_readback"] = (lambda: stats.absmean_var(big), big.numel() * 4)

    from torchmpi_b200 import config
    from torchmpi_b200.ops import gemm
    br, bc = (8192, 4096)
    bdy = torch.randn(br, bc, device=dev).to(torch.bfloat16)
    bz = torch.randn(br, bc, device=dev).to(torch.bfloat16)
    out["bias_grad_gelu_bwd"] = (lambda: gemm.bias_grad(bdy, bz), br * bc * 2 * 3)      # dy, z read; dz written
    out["bias_grad_plain"] = (lambda: gemm.bias_grad(bdy), br * bc * 2)
    bn_ = bdy[:, :1024].contiguous()
    out["bias_grad_plain_1024"] = (lambda: gemm.bias_grad(bn_), br * 1024 * 2)
    for name, (M, N, K) in {"gemm_bf16_8192": (8192, 8192, 8192), "gemm_bf16_tp_col": (8192, 4096, 8192),
                            "gemm_bf16_tp_row": (8192, 8192, 4096)}.items():
        if small and name != "gemm_bf16_tp_col":
            continue
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        b = torch.randn(N, K, device=dev).to(torch.bfloat16)
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        out[name] = (lambda a=a, b=b, c=c: gemm.matmul_nt(a, b, out=c), (M * K + N * K + M * N) * 2, 2.0 * M * N * K)

        def single(a=a, b=b, c=c):          # the 128 x 256 kernel on one CTA per tile
            config.set("gemm_pair", 0)
            try:
                gemm.matmul_nt(a, b, out=c)
            finally:
                config.set("gemm_pair", 1)
        out[name + "_1cta"] = (single, (M * K + N * K + M * N) * 2, 2.0 * M * N * K)
        if name == "gemm_bf16_tp_col":      # operands read as stored for dX = dY W and dW = dY^T X
            b_kn, a_km = b.t().contiguous(), a.t().contiguous()
            out[name + "_b_as_kn"] = (lambda a=a, b_kn=b_kn, c=c: gemm.matmul_nn(a, b_kn, out=c),
                                      (M * K + N * K + M * N) * 2, 2.0 * M * N * K)
            out[name + "_a_as_km_b_as_kn"] = (lambda a_km=a_km, b_kn=b_kn, c=c: gemm.matmul_tn(a_km, b_kn, out=c),
                                              (M * K + N * K + M * N) * 2, 2.0 * M * N * K)
        out[name + "_cublas"] = (lambda a=a, b=b, c=c: torch.matmul(a, b.t(), out=c), (M * K + N * K + M * N) * 2,
                                 2.0 * M * N * K)
    return out


def lazy_cases(small: bool) -> dict:
    """name -> builder; a builder allocates its inputs and returns ``(fn, bytes[, flops])``.  Built only when
    selected, so that a profiler capture of one kernel holds little memory."""
    import torch.nn.functional as F
    from torchmpi_b200.ops import conv, layernorm, pool
    from torchmpi_b200._lib import lib, dtype_code, stream_ptr, check
    dev = torch.device("cuda")
    B = 64 if small else 256
    out = {}

    def conv_case(hw, ci, co, k, stride, pad, mode):
        def build():
            x = torch.randn(B, ci, hw, hw, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            w = (torch.randn(co, ci, k, k, device=dev) * 0.05).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            y, _ = conv.conv_forward(x, w, stride, pad)
            dy = torch.randn_like(y)
            stats = torch.empty(lib.tmpi_conv_max_ctas() * 2 * co, dtype=torch.float32, device=dev)
            nx, ny, nw = x.numel() * 2, y.numel() * 2, w.numel() * 2
            flops = 2.0 * y.numel() * ci * k * k
            if mode == "fwd":
                return (lambda: conv.conv_forward(x, w, stride, pad)), nx + ny + nw, flops
            if mode == "fwd_stats":
                return (lambda: conv.conv_forward(x, w, stride, pad, stats)), nx + ny + nw, flops
            if mode == "dgrad":
                return (lambda: conv.conv_dgrad(dy, w, x.shape, 1, pad)), nx + ny + nw, flops
            if mode == "dgrad_add":
                other = torch.randn_like(x)
                return (lambda: conv.conv_dgrad(dy, w, x.shape, 1, pad, add=other)), 2 * nx + ny + nw, flops
            if mode == "wgrad":
                return (lambda: conv.conv_wgrad(dy, x, w.shape, stride, pad)), nx + ny + nw, flops
            if mode == "cudnn_fwd":
                return (lambda: F.conv2d(x, w, None, stride, pad)), nx + ny + nw, flops
            raise ValueError(mode)
        return build

    for tag, geom in {"1x1_56_64_256": (56, 64, 256, 1, 1, 0), "1x1_56_256_64": (56, 256, 64, 1, 1, 0),
                      "1x1_14_1024_256": (14, 1024, 256, 1, 1, 0), "3x3_56_64_64": (56, 64, 64, 3, 1, 1),
                      "3x3_14_256_256": (14, 256, 256, 3, 1, 1)}.items():
        for mode in ("fwd", "fwd_stats", "dgrad", "dgrad_add", "wgrad", "cudnn_fwd"):
            out[f"conv_{tag}_{mode}"] = conv_case(*geom, mode)

    def attn_case(own):
        def build():
            from torchmpi_b200.ops import attention
            Bq, T, H = (2 if small else 8), 1024, 16                      # GPT-2 medium: 16 heads of 64
            qkv = torch.randn(Bq, T, 3 * H * 64, device=dev).to(torch.bfloat16)
            flops = 4.0 * Bq * H * T * T * 64 / 2                          # causal: half of the score matrix
            nbytes = qkv.numel() * 2 + Bq * T * H * 64 * 2
            if own:
                return (lambda: attention.attention_forward(qkv, H)), nbytes, flops
            return (lambda: attention._reference(qkv, H)), nbytes, flops
        return build
    out["attention_fwd"] = attn_case(True)
    out["attention_sdpa_fwd"] = attn_case(False)

    def attn_bwd_case(route):
        def build():
            import math
            from torchmpi_b200.ops import attention
            Bq, T, H = (2 if small else 8), 1024, 16
            C = H * 64
            qkv = torch.randn(Bq, T, 3 * C, device=dev).to(torch.bfloat16)
            o, lse = attention.attention_forward(qkv, H)
            do = torch.randn_like(o)
            flops = 10.0 * Bq * H * T * T * 64 / 2                         # five products per block pair, causal
            nbytes = qkv.numel() * 2 * 2 + o.numel() * 2 * 2
            if route == "own":
                return (lambda: attention.attention_backward(qkv, o, lse, do, H)), nbytes, flops
            heads = lambda t: t.view(Bq, T, H, 64).transpose(1, 2)
            q, k, v = (heads(t) for t in qkv.split(C, dim=2))
            zero = torch.zeros((), dtype=torch.int64, device=dev)
            return (lambda: torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
                heads(do), q, k, v, heads(o), lse.unsqueeze(-1), zero, zero, None, None, None, T, T, 0.0, True,
                scale=1.0 / math.sqrt(64))), nbytes, flops
        return build
    out["attention_bwd"] = attn_bwd_case("own")
    out["attention_cudnn_bwd"] = attn_bwd_case("cudnn")

    def ln_case(backward):
        def build():
            rows, C = (131072 if not small else 65536), 1024        # > L2 both ways
            x = torch.randn(rows, C, device=dev).to(torch.bfloat16).requires_grad_(True)
            g = torch.ones(C, device=dev, dtype=torch.bfloat16, requires_grad=True)
            b = torch.zeros(C, device=dev, dtype=torch.bfloat16, requires_grad=True)
            if not backward:
                return (lambda: layernorm._LayerNormFn.apply(x.detach(), g.detach(), b.detach(), 1e-5)), rows * C * 2 * 2
            y = layernorm._LayerNormFn.apply(x, g, b, 1e-5)
            dy = torch.randn_like(y)
            return (lambda: torch.autograd.grad(y, (x, g, b), dy, retain_graph=True)), rows * C * 2 * 3
        return build
    out["layernorm_fwd"] = ln_case(False)
    out["layernorm_bwd"] = ln_case(True)

    def pool_case():
        N, C, H = (B, 64, 112)
        x = torch.randn(N, C, H, H, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last).requires_grad_(True)
        y = pool._MaxPoolFn.apply(x, 3, 2, 1)
        dy = torch.randn_like(y)
        return (lambda: torch.autograd.grad(y, x, dy, retain_graph=True)), (x.numel() + y.numel()) * 2 + y.numel()
    out["maxpool_bwd"] = pool_case

    def stem_case():
        x = torch.randn(B, 3, 224, 224, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        kpad = lib.tmpi_stem_patch_width()
        col = torch.empty((B * 112 * 112, kpad), dtype=torch.bfloat16, device=dev)
        def run():
            check(lib.tmpi_stem_im2col(x.data_ptr(), col.data_ptr(), B, 224, 224, dtype_code(x.dtype), stream_ptr()))
        return run, x.numel() * 2 + col.numel() * 2
    out["stem_im2col"] = stem_case

    # multi-rank kernels with a single member (no peer to wait for, so a profiler may replay them): the data
    # path of the two-shot allreduce and of the parameter-server push / pull on this GPU's own heap
    _heap = {}

    def heap():
        if "h" not in _heap:
            from torchmpi_b200.parallel.symm_heap import CudaHeap
            _heap["h"] = CudaHeap(0, 1, ((1 << 30) if small else (4 << 30)) + (256 << 20), 0)
        return _heap["h"]

    def twoshot_case():
        import ctypes as C
        from torchmpi_b200 import _lib
        h = heap()
        n = (64 if small else 256) << 20
        _, off_in = h.alloc(n * 2)
        _, off_out = h.alloc(n * 2)
        h.view(off_in, n * 2).view(torch.bfloat16).normal_()
        arr = _lib.int_array([0])
        g = _lib.Group(arr, 1, 0, 0)
        def run():
            check(lib.tmpi_cuda_allreduce_heap(off_in, off_out, n, 6, 1.0, C.byref(g), 2, stream_ptr()))
        run.keep = (arr, g)
        return run, n * 2 * 2
    out["coll_twoshot_one_member"] = twoshot_case

    def ps_case(rule):
        def build():
            h = heap()
            n = (64 if small else 256) << 20
            t = torch.randn(n, device=dev).to(torch.bfloat16)
            pid = h.ps_create(t, (0,))
            if rule < 0:
                return (lambda: h.ps_pull(pid, t).wait()), n * 2 * 2
            return (lambda: h.ps_push(pid, t, rule).wait()), n * 2 * (3 if rule == 2 else 2)
        return build
    out["ps_push_add_one_member"] = ps_case(2)
    out["ps_pull_one_member"] = ps_case(-1)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--small", action="store_true")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    peak, how = peak_gbs()
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")
    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    tf_peak = json.loads(f.read_text())["bf16_tflops"] if f.exists() else 1590.0
    lazy = lazy_cases(args.small)
    picked_lazy = {n: b for n, b in lazy.items() if args.kernel == "all" or n.startswith(args.kernel)}
    if args.kernel != "all" and picked_lazy:
        eager = {}                                   # a lazily built kernel was named: skip the eager set
    else:
        eager = cases(args.small)
    todo = [(n, c) for n, c in eager.items() if args.kernel == "all" or n.startswith(args.kernel)]
    todo += [(n, b()) for n, b in picked_lazy.items()]
    for name, case in todo:
        fn, nbytes = case[0], case[1]
        ms = time_kernel(fn, args.reps, flush)
        gbs = nbytes / ms / 1e6
        row = {"kernel": name, "bytes": nbytes, "ms": round(ms, 4), "gbs": round(gbs, 1),
               "frac_of_hbm_peak": round(gbs / peak, 3), "peak": how}
        if len(case) > 2:
            tf = case[2] / ms / 1e9
            row.update({"tflops": round(tf, 1), "frac_of_bf16_burst_peak": round(tf / tf_peak, 3)})
        print(json.dumps(row))


if __name__ == "__main__":
    main()
