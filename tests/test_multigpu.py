"""Real multi-GPU runs (one child process per GPU): peer-memory collectives over the symmetric heap,
the fused allreduce+SGD engine, the GPU parameter server, and a bounded-wait failure test.

The expected values follow test/collectives_all.lua (inputs filled with the rank) and
test/parameterserver.lua (the five scenarios).
"""
import os

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def world_sizes():
    n = ngpus()
    return [w for w in (2, 4, 8) if w <= n] or [2]


def all_world_sizes():
    """Every world size the collective matrix runs at: the powers of two and an odd one, as the reference loops
    over n = 2 .. GPUs (scripts/test_gpu.sh:47-50).  ``TORCHMPI_TEST_WORLDS=2,8`` narrows the list."""
    n = ngpus()
    env = os.environ.get("TORCHMPI_TEST_WORLDS")
    if env:
        return [int(w) for w in env.split(",") if int(w) <= max(n, 2)]
    return [w for w in (2, 3, 4, 8) if w <= n] or [2]


def _gather_equal(mpi, t):
    import torch.distributed as dist
    outs = [torch.empty_like(t) for _ in range(mpi.world_size())]
    dist.all_gather(outs, t.contiguous())
    for o in outs:
        assert torch.equal(o, outs[0]), "replicas differ"


def _collectives(rank, world, backend):
    os.environ["TORCHMPI_HEAP_BACKEND"] = backend
    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    config.set("device_wait_budget_ms", 5000)
    mpi.start(with_cuda=True)
    heap = mpi._S.cuda_heap
    assert heap is not None and heap.backend == (1 if backend == "vmm" else 0)
    dev = mpi.device
    n = world
    algos = ["auto", "oneshot", "twoshot", "ring"] + (["nvls"] if heap.has_multicast else [])
    info = {"multicast": heap.has_multicast}
    for dt in (torch.float32, torch.bfloat16, torch.int32, torch.float64):
        for size in (1, 255, 4096, 70001, 1 << 20, (1 << 22) + 8):
            for algo in algos:
                if algo == "nvls" and dt not in (torch.float32, torch.bfloat16):
                    continue
                t = torch.full((size,), rank, dtype=dt, device=dev)
                mpi.p2p.allreduce_tensor(t, algo=algo)
                assert torch.all(t == n * (n - 1) // 2), (dt, size, algo, t[:4].tolist())
            inp = torch.full((size,), rank, dtype=dt, device=dev)
            out = torch.full((size,), -1, dtype=dt, device=dev)
            mpi.allreduce_tensor(inp, out)
            assert torch.all(inp == rank) and torch.all(out == n * (n - 1) // 2)
            t = torch.full((size,), rank, dtype=dt, device=dev)
            mpi.broadcast_tensor(n - 1, t)
            assert torch.all(t == n - 1)
    heap.check_status(0)
    # random data against NCCL, and identical bits on every rank
    torch.manual_seed(100 + rank)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 4e-2)):
        for algo in algos:
            x = torch.randn(3_000_017, device=dev).to(dt)
            ref = x.clone()
            mpi.nccl.allreduce_tensor(ref)
            y = x.clone()
            mpi.p2p.allreduce_tensor(y, algo=algo, scale=0.25)
            assert torch.allclose(y.float(), ref.float() * 0.25, atol=tol * n, rtol=tol), (dt, algo)
            _gather_equal(mpi, y)
    # larger than the scratch region (several launches), and pointers whose alignment differs by rank
    big = torch.full((45_000_003,), float(rank + 1), device=dev)
    mpi.p2p.allreduce_tensor(big)
    assert torch.all(big == n * (n + 1) / 2)
    big.fill_(float(rank))
    mpi.p2p.broadcast_tensor(0, big)
    assert torch.all(big == 0)
    del big
    store = torch.full((100_004,), float(rank), device=dev)
    odd = store[rank % 2:][:100_000]
    mpi.p2p.allreduce_tensor(odd)
    assert torch.all(odd == n * (n - 1) / 2)
    odd.fill_(float(rank))
    mpi.p2p.broadcast_tensor(n - 1, odd)
    assert torch.all(odd == n - 1)
    heap.check_status(0)
    # tensors living in the symmetric heap take the zero-copy path
    sym = heap.empty(1 << 20, torch.bfloat16)
    sym.fill_(rank + 1)
    mpi.p2p.allreduce_tensor(sym)
    assert torch.all(sym == n * (n + 1) // 2)
    # every broadcast algorithm on a heap tensor whose length does not split evenly (pull, scatter + all-gather,
    # multicast store, scatter + multicast stores, scatter + plain stores; the multicast ones fall back to the pull
    # without a mapping)
    symb = heap.empty((1 << 20) + 8 * 13, torch.bfloat16)
    for algo in (1, 2, 3, 4, 5):
        mpi.config.set("broadcast_algo", algo)
        for root in (0, n - 1):
            symb.copy_((torch.arange(symb.numel(), device=dev) % 251 + rank * 7).to(torch.bfloat16))
            mpi.p2p.broadcast_tensor(root, symb)
            expect = (torch.arange(symb.numel(), device=dev) % 251 + root * 7).to(torch.bfloat16)
            assert torch.equal(symb, expect), (algo, root)
    mpi.config.set("broadcast_algo", 0)
    heap.check_status(0)
    # reduce / allgather(v) / reduce_scatter / sendreceive
    for size in (7, 4096, 1 << 18):
        inp = torch.full((size,), float(rank), device=dev)
        out = torch.full((size,), -1.0, device=dev)
        mpi.p2p.reduce_tensor(0, inp, out)
        assert torch.all(out == (n * (n - 1) / 2 if rank == 0 else -1.0))
    inp = torch.full((5 + rank,), float(rank), device=dev)
    res = mpi.p2p.allgather_tensor(inp, torch.empty(1, device=dev))
    expect = torch.cat([torch.full((5 + r,), float(r)) for r in range(n)]).to(dev)
    assert torch.equal(res.view(-1), expect)
    inp = (torch.arange(n * 4096, dtype=torch.float32) + rank).to(dev)
    out = torch.empty(4096, device=dev)
    mpi.reduce_scatter_tensor(inp, out)
    base = torch.arange(rank * 4096, (rank + 1) * 4096, dtype=torch.float32, device=dev)
    assert torch.equal(out, base * n + n * (n - 1) / 2)
    t = torch.full((1000,), float(rank), device=dev)
    mpi.sendreceive_tensor(t, (rank - 1) % n, (rank + 1) % n)
    assert torch.all(t == (rank - 1) % n)
    # async handles: launch returns at once, device-side and host-side joins
    import time
    hs, ts = [], []
    for i in range(6):
        t = torch.full((1 << 18,), float(rank + i), device=dev)
        t0 = time.perf_counter()
        hs.append(mpi.async_.p2p.allreduce_tensor(t))
        info.setdefault("launch_us", []).append((time.perf_counter() - t0) * 1e6)
        ts.append(t)
    for i, (h, t) in enumerate(zip(hs, ts)):
        h.wait_stream()
        mpi.sync_handle(h)
        assert torch.all(t == n * (n - 1) / 2 + n * i)
    h = mpi.async_.p2p.broadcast_tensor(0, ts[0])
    mpi.sync_handle(h)
    heap.check_status(1)
    mpi.check_with_allreduce(ts[0], "broadcast result")
    mpi.barrier()
    mpi.stop()
    return info


@pytest.mark.parametrize("world", all_world_sizes())
@pytest.mark.parametrize("backend", ["ipc", "vmm"])
def test_gpu_collectives(backend, world):
    res = run_ranks(_collectives, world, backend, timeout=600)
    print(backend, world, res[0])


def _hierarchical(rank, world):
    """Hierarchical allreduce on GPUs (groups pushed as a second communicator level, lib/collectives_cuda.cpp:501-581):
    synchronous, asynchronous (a live handle at once, the whole intra -> inter -> broadcast chain behind it,
    lib/collectives_cuda.cpp:771-803) and from the asynchronous backward registration, each equal to the flat result."""
    import time
    import torchmpi_b200 as mpi
    from torchmpi_b200 import nn as mpinn
    gsize = 2 if world >= 4 else 1

    def custom():
        return mpi.push_communicator(str(mpi.rank() // gsize))

    mpi.start(with_cuda=True, custom_communicator_init=custom, with_cartesian_communicator=True)
    dev = mpi.device
    mpi.set_collective_span(0, 1)                  # outer = everyone, inner = the groups
    want = world * (world - 1) / 2
    for n in (1000, 1 << 20):
        t = torch.full((n,), float(rank), device=dev)
        mpi.allreduce_tensor(t)
        assert torch.all(t == want), (n, t[:3])
        mpi.config.set_flat_collectives()
        f = torch.full((n,), float(rank), device=dev)
        mpi.allreduce_tensor(f)
        assert torch.equal(f, t)
        mpi.config.set_hierarchical_collectives()
        a = torch.full((n,), float(rank), device=dev)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        h = mpi.async_.allreduce_tensor(a)
        launch_us = (time.perf_counter() - t0) * 1e6
        assert h is not None and launch_us < 20000, launch_us       # returns at once: the chain runs behind the handle
        mpi.sync_handle(h)
        torch.cuda.synchronize()
        assert torch.equal(a, t)
    # gradients through the asynchronous backward registration on the hierarchical span
    torch.manual_seed(7)
    net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10)).to(dev)
    mpinn.synchronize_parameters(net)
    x = torch.randn(32, 64, generator=torch.Generator().manual_seed(100 + rank)).to(dev)
    mpinn.async_.register_async_mpi_backward(net, scale=1.0 / world)
    net(x).square().mean().backward()
    mpinn.async_.synchronize_gradients(net)
    torch.cuda.synchronize()
    got = [p.grad.clone() for p in net.parameters()]
    mpinn.async_.unregister_async_mpi_backward(net)
    net.zero_grad()
    net(x).square().mean().backward()
    mpi.config.set_flat_collectives()
    mpinn.synchronize_gradients(net, scale=1.0 / world)
    for g, p in zip(got, net.parameters()):
        assert torch.allclose(g, p.grad, atol=1e-6, rtol=1e-5)
    mpi.stop()
    return True


def test_hierarchical_allreduce_on_gpus():
    # two ranks, groups of one: the whole chain (intra, inter, broadcast) with the smallest GPU count; groups of two
    # run among CPU ranks (tests/test_cpu_collectives.py) and in the 2 x 4 GPT-2 benchmark
    assert all(run_ranks(_hierarchical, 2, timeout=600))


def _engine(rank, world):
    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    from torchmpi_b200.engine import AllReduceSGDEngine
    from torchmpi_b200.models import resnet, to_bf16_mixed
    from torchmpi_b200.ops import xent
    config.set("device_wait_budget_ms", 5000)
    mpi.start(with_cuda=True)
    dev = mpi.device
    torch.manual_seed(10 + rank)            # different init per rank; the engine broadcasts rank 0's
    model = to_bf16_mixed(resnet.resnet_tiny(10, fused_bn=True).to(dev)).to(memory_format=torch.channels_last)
    g = torch.Generator().manual_seed(50 + rank)
    batches = [{"input": torch.randn(16, 3, 64, 64, generator=g).to(torch.bfloat16).to(dev)
                .contiguous(memory_format=torch.channels_last),
                "target": torch.randint(0, 10, (16,), generator=g).to(dev)} for _ in range(4)]
    engine = AllReduceSGDEngine(usegpu=True, devicesync=False, fused=True, momentum=0.9,
                                gradient_scale=1.0 / world, bucket_bytes=128 << 10)
    losses = []
    engine.hooks["onUpdate"] = lambda st: losses.append(float(st["loss"].detach()))
    engine.train(model, xent.CrossEntropyLoss(), batches, lr=0.05, maxepoch=5)
    torch.cuda.synchronize()
    engine._opt.check()
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    _gather_equal(mpi, flat)
    assert torch.isfinite(flat).all()
    sd = engine._opt.state_dict()           # collective: gathers the sharded fp32 state
    assert sd["step"] == 20 and sd["buckets"][0]["momentum"] is not None
    mpi.stop()
    return losses


def test_fused_engine_data_parallel():
    world = world_sizes()[-1]
    res = run_ranks(_engine, world, timeout=600)
    first = sum(r[0] for r in res) / world
    last = sum(r[-1] for r in res) / world
    assert last < first, (first, last)       # the fixed batches are being fitted


def _ps(rank, world):
    import torchmpi_b200 as mpi
    from torchmpi_b200 import parameterserver as ps
    mpi.start(with_cuda=True)
    dev = mpi.device
    n = world
    for it in range(5):
        # (1) default init: every rank's own shard survives a round trip
        t = torch.full((1000,), float(rank), device=dev)
        server = ps.init(t)
        assert server.on_gpu
        out = torch.empty_like(t)
        mpi.sync_handle(ps.receive(server, out))
        for r in range(n):
            b, e = ps.shard_range(1000, n, r)
            assert torch.all(out[b:e] == r)
        ps.free(server)
        # (2) a 2-D tensor, 911 x 101
        t2 = torch.full((911, 101), float(rank), device=dev)
        server = ps.init(t2)
        # (3) zero from the last rank, barrier, everybody receives zeros
        if rank == n - 1:
            mpi.sync_handle(ps.send(server, t2, "zero"))
        mpi.barrier()
        out2 = torch.empty_like(t2)
        mpi.sync_handle(ps.receive(server, out2))
        assert torch.all(out2 == 0)
        mpi.barrier()
        # (4) copy from the last rank
        if rank == n - 1:
            mpi.sync_handle(ps.send(server, t2, "copy"))
        mpi.barrier()
        mpi.sync_handle(ps.receive(server, out2))
        assert torch.all(out2 == n - 1)
        mpi.barrier()
        # (5) everybody adds its rank: n-1 + n(n-1)/2
        mpi.sync_handle(ps.send(server, t2, "add"))
        mpi.barrier()
        mpi.sync_handle(ps.receive(server, out2))
        assert torch.all(out2 == n - 1 + n * (n - 1) / 2), out2.flatten()[:4]
        ps.free(server)
    # the parameter server used as an allreduce (zero / add / receive / divide)
    torch.manual_seed(3 + rank)
    x = torch.randn(100_003, device=dev)
    ref = x.clone()
    mpi.nccl.allreduce_tensor(ref)
    server = ps.init(x)
    if rank == 0:
        mpi.sync_handle(ps.send(server, x, "zero"))
    mpi.barrier()
    mpi.sync_handle(ps.send(server, x, "add"))
    mpi.barrier()
    got = torch.empty_like(x)
    mpi.sync_handle(ps.receive(server, got))
    assert torch.allclose(got, ref, atol=1e-4, rtol=1e-5)
    ps.free_all()
    mpi.stop()
    return True


def test_gpu_parameter_server():
    assert all(run_ranks(_ps, world_sizes()[0], timeout=600))


def _absent_peer(rank, world):
    """Rank 1 never launches its kernel: rank 0's bounded device wait must report a timeout, and
    the context must stay usable.  NVLS is off and the heap uses plain peer mappings."""
    os.environ["TORCHMPI_HEAP_BACKEND"] = "ipc"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    config.set("device_wait_budget_ms", 1000)
    config.set("device_wait_startup_grace_ms", 0)      # the steady-state budget from the first call on
    config.set("use_nvls", 0)
    mpi.start(with_cuda=True)
    dev = mpi.device
    t = torch.ones(1 << 16, device=dev)
    mpi.p2p.allreduce_tensor(t)              # a healthy collective first
    torch.cuda.synchronize()
    mpi.barrier()
    outcome = "skipped"
    from torch.distributed import distributed_c10d
    store = distributed_c10d._get_default_store()
    if rank == 0:
        mpi.p2p.allreduce_tensor(t)          # nobody answers
        torch.cuda.synchronize()
        try:
            mpi._S.cuda_heap.check_status(0)
            outcome = "no error"
        except mpi.TimeoutError as e:
            outcome = "timeout: " + str(e)
        assert float(torch.ones(8, device=dev).sum()) == 8.0     # context still answers
        try:                                  # the job is poisoned: the next collective fails at once
            mpi.p2p.allreduce_tensor(t)
            outcome += " / not poisoned"
        except mpi.CommunicatorPoisoned:
            pass
        store.set("tmpi_test/absent_peer_done", "1")
    else:
        store.get("tmpi_test/absent_peer_done")                  # learns of the failure on the host, launches nothing
        mpi.watchdog.poison("rank 0 reported a failed collective")
    mpi.stop()                               # both ranks leave between steps, nothing in flight, no barrier
    return outcome


def test_bounded_wait_when_peer_never_launches():
    res = run_ranks(_absent_peer, 2, timeout=300)
    assert res[0].startswith("timeout"), res


def _tp_mlp(rank, world):
    """Tensor-parallel MLP (fused all-gather->GEMM, GEMM->reduce-scatter) against the unsharded model."""
    import math
    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    from torchmpi_b200.parallel.tensor_parallel import TensorParallelMLP, TensorParallelMLPBlock
    config.set("device_wait_budget_ms", 5000)
    mpi.start(with_cuda=True)
    dev = mpi.device
    rows, D, F = 256, 512, 2048
    M = rows * world
    model = TensorParallelMLP(rows, d_model=D, d_hidden=F, layers=4, bias=True)
    f = F // world
    # rebuild the unsharded weights from the per-slice seeds
    w1 = torch.empty(2, F, D)
    w2 = torch.empty(2, D, F)
    for b in range(2):
        for r in range(world):
            g = torch.Generator().manual_seed(TensorParallelMLPBlock.slice_seed(r, F))
            w1[b, r * f:(r + 1) * f] = torch.randn(f, D, generator=g) / math.sqrt(D)
            w2[b, :, r * f:(r + 1) * f] = torch.randn(D, f, generator=g) / math.sqrt(F)
    w1, w2 = w1.to(dev).to(torch.bfloat16).float(), w2.to(dev).to(torch.bfloat16).float()
    gx = torch.Generator().manual_seed(99)
    x_full = torch.randn(M, D, generator=gx).to(dev).to(torch.bfloat16)
    dy_full = torch.randn(M, D, generator=gx).to(dev).to(torch.bfloat16)
    xs = x_full[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    for rep in range(2):
        y = model(xs)
        y.backward(dy_full[rank * rows:(rank + 1) * rows])
    torch.cuda.synchronize()
    model.tp.check()
    # reference in fp32 on the gathered data (two passes accumulate the gradients twice)
    xr = x_full.float().requires_grad_(True)
    p1 = [w1[b].clone().requires_grad_(True) for b in range(2)]
    p2 = [w2[b].clone().requires_grad_(True) for b in range(2)]
    h = xr
    for b in range(2):
        h = torch.nn.functional.gelu(h @ p1[b].t()) @ p2[b].t()
    h.backward(dy_full.float())
    sl = slice(rank * rows, (rank + 1) * rows)
    assert torch.allclose(y.float(), h[sl], rtol=5e-2, atol=5e-2), (y.float() - h[sl]).abs().max()
    assert torch.allclose(xs.grad.float(), 2 * xr.grad[sl], rtol=5e-2, atol=5e-2)
    blk = model[0]

    def rel(a, b):       # bf16 operands and a bf16 result: compare in the Frobenius norm
        return ((a - b).norm() / b.norm()).item()
    assert rel(blk.w1.grad.float(), 2 * p1[0].grad[rank * f:(rank + 1) * f]) < 0.02
    assert rel(blk.w2.grad.float(), 2 * p2[0].grad[:, rank * f:(rank + 1) * f]) < 0.02
    assert rel(model[1].w2.grad.float(), 2 * p2[1].grad[:, rank * f:(rank + 1) * f]) < 0.02
    mpi.stop()
    return True


def test_tensor_parallel_mlp():
    assert all(run_ranks(_tp_mlp, world_sizes()[-1], timeout=600))
