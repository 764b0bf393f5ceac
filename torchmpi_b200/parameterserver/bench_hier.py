"""Hierarchical asynchronous training benchmark: sync fused allreduce inside groups, EASGD across them.

    python -m torch.distributed.run --nproc-per-node 8 -m torchmpi_b200.parameterserver.bench_hier \
        [--group-size 4] [--model gpt2_medium] [--batch 8] [--steps 20] [--warmup 4] [--update-frequency 4]

The GPUs form ``world / group_size`` groups.  Inside a group every step ends with the fused
allreduce+SGD kernel over the group's ranks.  Across groups the parameters are kept loosely together
by a GPU-resident parameter server sharded over ALL ranks: every ``update_frequency`` steps the root
of each group pulls the centre (prefetched two steps earlier, overlapped with compute), applies the
elastic update, pushes its delta back and broadcasts the result inside its group - the scheme of
examples/mnist/mnist_parameterserver_easgd_dataparallel.lua:28-35,67-91 on GPT-2.
Prints tokens/s (device-timed, max over ranks) and the bandwidth of a stand-alone push and pull of the
whole parameter vector.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--group-size", type=int, default=4)
    ap.add_argument("--model", default="gpt2_medium", choices=["gpt2_medium", "gpt2_tiny"])
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--update-frequency", type=int, default=4)
    ap.add_argument("--tc-linear", type=int, default=1)
    ap.add_argument("--profile-one-step", action="store_true",
                    help="after the warm-up run one step between cudaProfilerStart/Stop and exit (no timing)")
    args = ap.parse_args()

    import torchmpi_b200 as mpi
    from torchmpi_b200 import config, parameterserver as ps
    from torchmpi_b200.engine import AllReduceSGDEngine
    from torchmpi_b200.models import gpt2
    config.set("heap_bytes", 6 << 30)

    def groups():
        return mpi.push_communicator(str(mpi.rank() // args.group_size))

    mpi.start(with_cuda=True, custom_communicator_init=groups)
    mpi.set_collective_span(1, 1)                    # tensor collectives act inside a group
    mpi.set_communicator(0)
    rank, world, dev = mpi.world_rank(), mpi.world_size(), mpi.device
    torch.manual_seed(1)
    model = (gpt2.gpt2_medium(tc_linear=bool(args.tc_linear)) if args.model == "gpt2_medium"
             else gpt2.gpt2_tiny(tc_linear=bool(args.tc_linear), block_size=args.seq))
    model = model.to(dev).to(torch.bfloat16)
    seq = min(args.seq, model.config.block_size)
    vocab = model.config.vocab_size
    nparams = sum(p.numel() for p in model.parameters())
    g = torch.Generator().manual_seed(100 + rank)
    data = [(torch.randint(0, vocab, (args.batch, seq), generator=g).to(dev),
             torch.randint(0, vocab, (args.batch, seq), generator=g).to(dev)) for _ in range(4)]

    group = mpi.intra_members(1)
    engine = AllReduceSGDEngine(usegpu=True, devicesync=False, fused=True, momentum=0.9,
                                gradient_scale=1.0 / len(group))
    criterion = gpt2.LMLoss(unit_grad=True)          # the engine calls backward on this loss itself
    state = {"network": model, "criterion": criterion, "iterator": None, "lr": 1e-3, "lrcriterion": 0.0,
             "maxepoch": 1, "sample": None, "epoch": 0, "t": 0, "training": True}
    engine._setup(model, criterion)
    model.train()
    updater = ps.EASGDUpdate(model, sharding_communicator=0, dataparallel_communicator=1, beta=0.9,
                             update_frequency=args.update_frequency, init_delay=1, prefetch=args.update_frequency - 2
                             if args.update_frequency > 2 else 0)
    updater.on_parameters_changed = engine._opt.refresh_master

    def step(i):
        x, y = data[i % len(data)]
        engine.train_step(state, {"input": x, "target": y})
        updater.update(state["t"])

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    mpi.barrier()
    if args.profile_one_step:
        # for `ncu --profile-from-start off`: exactly one training step lies inside the profiler range
        torch.cuda.profiler.start()
        step(args.warmup)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        mpi.stop()
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / args.steps
    engine._opt.check()

    # stand-alone push / pull of the whole (flat) parameter vector through the parameter server
    flat = torch.cat([b.reshape(-1) for b in engine._opt.buckets.weight_blocks()]).contiguous()
    server = ps.init(flat)
    upd = torch.zeros_like(flat)
    res = {}
    for name, fn in (("push_add", lambda: server.send(upd, "add")), ("pull", lambda: server.receive(flat))):
        for _ in range(2):
            fn().wait()
        torch.cuda.synchronize()
        mpi.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        hs = [fn() for _ in range(5)]
        for h in hs:
            h.wait_stream()
        b.record()
        for h in hs:
            h.wait()
        torch.cuda.synchronize()
        tt = torch.tensor([a.elapsed_time(b) / 5], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        moved = flat.numel() * flat.element_size() * (world - 1) / world     # bytes that cross NVLink per rank
        res[name] = {"ms": tt.item(), "gbs": moved / tt.item() / 1e6, "roofline_frac": moved / tt.item() / 1e6 / 770.0}
    ps.free(server)
    out = {"metric": "GPT-2 hierarchical async training tokens/s", "value": world * args.batch * seq / (ms / 1e3),
           "unit": "tokens/s", "ms_per_step": ms, "n_gpus": world,
           "config": {"model": args.model, "params": nparams, "groups": world // args.group_size,
                      "group_size": args.group_size, "batch_per_gpu": args.batch, "seq": seq,
                      "update_frequency": args.update_frequency, "dtype": "bf16",
                      "data": "synthetic uniform token ids, random-init weights"},
           "parameter_server": res}
    if rank == 0:
        print(json.dumps(out))
    mpi.stop()


if __name__ == "__main__":
    main()
