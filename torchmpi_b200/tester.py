"""Correctness and bandwidth sweeps of the collectives (reference: torchmpi/tester.lua, test/collectives_all.lua).

``python -m torch.distributed.run --nproc-per-node N -m torchmpi_b200.tester [options]``

For every collective, dtype, backend/algorithm and size (powers of two from ``--min-bytes`` to
``--max-bytes``) the tensor is filled with the rank, the collective is checked on its first run
(allreduce / reduce must give n(n-1)/2, broadcast the root's rank, allgather the rank-ordered
concatenation), and then timed.  Unlike the reference, which wraps a host timer around two MPI
barriers (torchmpi/tester.lua:61-96), timing is on the device: CUDA events on the launching stream
around ``--iters`` back-to-back launches after ``--warmup`` untimed ones, maximum over ranks.
Bandwidths use the reference's formulas (test/collectives_all.lua:215-218,261-264,454-457):
allreduce busBW = 2 S (n-1)/n / t;  broadcast, reduce = S / t;  allgather = S_in (n-1) / t;
reduce_scatter = S_out (n-1) / t.  Each row also carries the fraction of the NVLink roofline
(``--link-gbs``, default the measured 770 GB/s per direction).  Rank 0 prints one JSON object per row.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "int32": torch.int32,
          "fp64": torch.float64}


def bus_bw(op: str, nbytes: int, n: int, seconds: float) -> float:
    """GB/s by the reference's formulas; ``nbytes`` is the per-rank message (output slice for reduce_scatter)."""
    if op == "allreduce":
        return 2 * nbytes * (n - 1) / n / seconds / 1e9
    if op in ("allgather", "reduce_scatter"):
        return nbytes * (n - 1) / seconds / 1e9
    return nbytes / seconds / 1e9


def roofline_bus_bw(op: str, variant: str, n: int, link: float) -> float:
    """Upper bound on the figure ``bus_bw`` can reach, given ``link`` GB/s per direction per GPU."""
    if op == "allreduce":
        if variant == "oneshot":
            return 2 * link / n                       # every rank receives (n-1) S
        if variant == "nvls":
            return 2 * (n - 1) / (n + 1) * link       # (1 + 1/n) S per direction
        return link                                   # two-shot / ring: 2 (n-1)/n S
    return link       # broadcast (S / B with a multicast store), reduce, all-gather, reduce-scatter


def _timed(fn, warmup: int, iters: int, device_timing: bool) -> float:
    for _ in range(warmup):
        fn()
    if device_timing:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 1e3 / iters], dtype=torch.float64)
    else:
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        t = torch.tensor([(time.perf_counter() - t0) / iters], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def run(args) -> list:
    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    use_gpu = args.processor == "gpu"
    if use_gpu:
        # the largest symmetric tensor is the reduce-scatter input: world x max_bytes
        import os
        nranks = int(os.environ.get("WORLD_SIZE", "1")) if "reduce_scatter" in args.ops else 1
        config.set("heap_bytes", max(config.get("heap_bytes"), (nranks + 3) * args.max_bytes + (256 << 20)))
        config.set("staging_bytes", max(config.get("staging_bytes"), min(args.max_bytes, 1 << 30)))
        if args.ctas:
            config.set("comm_max_ctas", args.ctas)
    for kv in args.set:
        name, _, value = kv.partition("=")
        config.set(name, int(value))
    mpi.start(with_cuda=use_gpu, with_cartesian_communicator=args.cartesian)
    rank, n, dev = mpi.rank(), mpi.size(), mpi.device
    heap = mpi._S.cuda_heap
    rows = []
    ops = args.ops.split(",")
    variants = args.variants.split(",")
    sizes, b = [], args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 2
    for op in ops:
        for dname in args.dtypes.split(","):
            dt = DTYPES[dname]
            es = torch.empty((), dtype=dt).element_size()
            for variant in variants:
                if variant == "nvls" and not (use_gpu and heap is not None and heap.has_multicast):
                    continue
                if variant in ("oneshot", "twoshot", "nvls", "ring") and op not in ("allreduce",):
                    if not (op == "broadcast" and variant in ("nvls",)):
                        continue
                for nbytes in sizes:
                    numel = max(1, nbytes // es)
                    if variant == "oneshot" and nbytes > config.get("oneshot_max_bytes"):
                        continue
                    backend = "nccl" if variant == "nccl" else ("gloo" if variant == "gloo" else "p2p")
                    algo = variant if variant in ("oneshot", "twoshot", "nvls", "ring") else "auto"
                    if args.symmetric and use_gpu and backend == "p2p":
                        heap_mark = heap.alloc(0)[1]
                        t = heap.empty(numel * (n if op == "reduce_scatter" else 1), dt)
                    else:
                        heap_mark = None
                        t = torch.empty(numel * (n if op == "reduce_scatter" else 1), dtype=dt, device=dev)
                    out = torch.empty(numel * (n if op == "allgather" else 1), dtype=dt, device=dev)

                    def call():
                        if op == "allreduce":
                            mpi.allreduce_tensor(t, backend=backend, algo=algo)
                        elif op == "broadcast":
                            mpi.broadcast_tensor(0, t, backend=backend)
                        elif op == "reduce":
                            mpi.reduce_tensor(0, t, out, backend=backend)
                        elif op == "allgather":
                            mpi.allgather_tensor(t, out, backend=backend, equal_counts=args.benchmark)
                        elif op == "reduce_scatter":
                            mpi.reduce_scatter_tensor(t, out, backend=backend)
                    # correctness on the first run
                    t.fill_(rank)
                    call()
                    if use_gpu:
                        torch.cuda.synchronize()
                    ok = True
                    if op == "allreduce":
                        ok = bool(torch.all(t == n * (n - 1) // 2))
                    elif op == "broadcast":
                        ok = bool(torch.all(t == 0))
                    elif op == "reduce" and rank == 0:
                        ok = bool(torch.all(out == n * (n - 1) // 2))
                    elif op == "allgather":
                        ok = all(bool(torch.all(out[r * numel:(r + 1) * numel] == r)) for r in range(n))
                    elif op == "reduce_scatter":
                        ok = bool(torch.all(out == n * (n - 1) // 2))
                    if not ok:
                        raise AssertionError(f"{op} {variant} {dname} {nbytes} B: wrong result on rank {rank}")
                    if args.benchmark:
                        t.zero_()
                        iters = args.iters if nbytes <= (64 << 20) else max(3, args.iters // 4)
                        sec = _timed(call, args.warmup, iters, use_gpu)
                        bw = bus_bw(op, numel * es, n, sec)
                        roof = roofline_bus_bw(op, variant, n, args.link_gbs)
                        row = {"op": op, "variant": variant, "dtype": dname, "bytes": numel * es, "world": n,
                               "us": round(sec * 1e6, 2), "alg_gbs": round(numel * es / sec / 1e9, 2),
                               "bus_gbs": round(bw, 2), "roofline_frac": round(bw / roof, 3),
                               "roofline_frac_900": round(bw / roofline_bus_bw(op, variant, n, 900.0), 3),
                               "symmetric": bool(args.symmetric)}
                        if args.tag:
                            row["tag"] = args.tag
                        rows.append(row)
                        if rank == 0:
                            print(json.dumps(row), flush=True)
                    del t, out
                    if heap_mark is not None:
                        from torchmpi_b200._lib import lib
                        lib.tmpi_cuda_heap_reset_allocator(heap_mark)
    if use_gpu and heap is not None:
        heap.check_status(0)
    mpi.barrier()
    if rank == 0 and not args.benchmark:
        print("Success")
    mpi.stop()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--processor", default="gpu" if torch.cuda.is_available() else "cpu", choices=["cpu", "gpu"])
    ap.add_argument("--ops", default="allreduce,broadcast,reduce_scatter,allgather")
    ap.add_argument("--variants", default="auto,oneshot,twoshot,nvls,ring,nccl")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--min-bytes", type=int, default=4 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--benchmark", action="store_true")
    ap.add_argument("--symmetric", action="store_true", help="place the tensors in the symmetric heap (zero-copy path)")
    ap.add_argument("--cartesian", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ctas", type=int, default=0, help="CTAs per collective kernel (default: the comm_max_ctas tunable)")
    ap.add_argument("--link-gbs", type=float, default=770.0,
                    help="measured per-direction link rate for roofline_frac (the nominal 900 GB/s is reported beside it)")
    ap.add_argument("--set", action="append", default=[], metavar="NAME=VALUE", help="set a runtime tunable (sweeps)")
    ap.add_argument("--tag", default="", help="copied into every result row")
    run(ap.parse_args())


if __name__ == "__main__":
    main()
