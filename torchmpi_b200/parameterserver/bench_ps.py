"""Bandwidth of the one-sided GPU parameter-server kernels (push with each rule, pull) against size.

    python -m torch.distributed.run --nproc-per-node 8 -m torchmpi_b200.parameterserver.bench_ps \
        [--min-bytes 1048576] [--max-bytes 1073741824] [--dtype bf16] [--ctas 0]

Every rank is a client of a server sharded over all ranks and issues the same request at the same
time (the all-to-all pattern of a synchronous step).  Device-timed with CUDA events on the launching
stream, 3 warm-up requests, max over ranks; tensors of 256 MiB and more exceed the L2.  ``gbs`` counts
the bytes that cross NVLink per rank, ``(world - 1) / world`` of the tensor; the roofline is the link
rate per direction.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1 << 20)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", type=int, default=0, help="CTAs per kernel (default: the ps_max_ctas tunable)")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()

    import torchmpi_b200 as mpi
    from torchmpi_b200 import config, parameterserver as ps
    config.set("heap_bytes", 2 * args.max_bytes + (512 << 20))
    if args.ctas:
        config.set("ps_max_ctas", args.ctas)
    mpi.start(with_cuda=True)
    rank, world, dev = mpi.rank(), mpi.size(), mpi.device
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    es = 2 if args.dtype == "bf16" else 4
    size = args.min_bytes
    while size <= args.max_bytes:
        t = torch.randn(size // es, device=dev).to(dt)
        server = ps.init(t)
        for name, fn in (("push_copy", lambda: server.send(t, "copy")), ("push_add", lambda: server.send(t, "add")),
                         ("pull", lambda: server.receive(t))):
            for _ in range(3):
                fn().wait()
            torch.cuda.synchronize()
            mpi.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            hs = [fn() for _ in range(args.iters)]
            for h in hs:
                h.wait_stream()
            b.record()
            for h in hs:
                h.wait()
            torch.cuda.synchronize()
            ms = torch.tensor([a.elapsed_time(b) / args.iters], dtype=torch.float64)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            moved = size * (world - 1) / world
            if rank == 0:
                print(json.dumps({"op": name, "dtype": args.dtype, "bytes": size, "world": world,
                                  "us": round(ms.item() * 1e3, 2), "gbs": round(moved / ms.item() / 1e6, 1),
                                  "roofline_frac": round(moved / ms.item() / 1e6 / args.link_gbs, 3),
                                  "ctas": config.get("ps_max_ctas")}), flush=True)
        ps.free(server)
        del t
        size *= 4
    mpi.stop()


if __name__ == "__main__":
    main()
