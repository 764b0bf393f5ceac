"""Multi-rank kernels on ONE GPU: every rank's slab lives on the same device and one cooperative
launch (gridDim.y = ranks) runs all ranks of a collective, so the flag protocol, the shard arithmetic
and the reductions are exercised without a second GPU.  Oracle: fp64 sums computed by PyTorch.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.float32: 7, torch.bfloat16: 6, torch.float16: 5, torch.float64: 8, torch.int32: 3, torch.int64: 4,
      torch.int8: 1}


@pytest.fixture(scope="module", params=[2, 4, 8])
def emu(request):
    from torchmpi_b200 import config
    from torchmpi_b200.parallel.symm_heap import CudaHeap
    torch.cuda.set_device(0)
    config.set("device_wait_budget_ms", 2000)
    h = CudaHeap(0, request.param, 96 << 20, 0, emulated=True)
    yield h
    torch.cuda.synchronize()
    h.destroy()


def group(world, lane=0):
    from torchmpi_b200 import _lib
    arr = _lib.int_array(range(world))
    return _lib.Group(arr, world, 0, lane), arr


def fill(h, n, dtype, seed):
    """Allocates a symmetric buffer and fills rank r's copy with seeded data; returns (offset, [tensors])."""
    es = torch.empty((), dtype=dtype).element_size()
    _, off = h.alloc(n * es)
    ts = []
    g = torch.Generator(device="cuda").manual_seed(seed)
    for r in range(h.world):
        t = h.view(off, n * es, peer=r).view(dtype)
        if dtype.is_floating_point:
            t.copy_(torch.randn(n, generator=g, device="cuda", dtype=torch.float32).to(dtype))
        else:
            t.copy_(torch.randint(-50, 50, (n,), generator=g, device="cuda").to(dtype))
        ts.append(t)
    return off, ts


def status_ok(h):
    h.check_status(0)


@pytest.mark.parametrize("algo", [1, 2, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64, torch.int32, torch.int8])
def test_allreduce_variants(emu, algo, dtype):
    from torchmpi_b200._lib import lib, check
    h, W = emu, emu.world
    lib.tmpi_cuda_heap_reset_allocator(0)
    for n in ([16, 1000, 65536] if algo == 1 else [16 * W, 4096 + 16 * W, 1 << 20]):
        if algo == 1 and n * torch.empty((), dtype=dtype).element_size() > (512 << 10):
            continue
        in_off, ins = fill(h, n, dtype, 1)
        ref = sum(t.double() for t in ins)
        scale = 0.5 if dtype.is_floating_point else 1.0
        if algo == 4:
            out_off, outs = in_off, ins
        else:
            out_off, outs = fill(h, n, dtype, 2)
        g, keep = group(W)
        check(lib.tmpi_cuda_allreduce_heap(in_off, out_off, n, DT[dtype], scale, C.byref(g), algo,
                                           torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        status_ok(h)
        want = (ref * scale)
        tol = {torch.bfloat16: 0.08 * W ** 0.5, torch.float16: 0.02, torch.float32: 1e-4,
               torch.float64: 1e-12}.get(dtype, 0)
        for r in range(W):
            got = outs[r].double()
            assert torch.allclose(got, want.to(dtype).double() if tol == 0 else want, atol=tol, rtol=tol), (algo, dtype, n, r)
            assert torch.equal(outs[r], outs[0]), "replicas must hold identical bits"


def test_allreduce_rank_fill_is_exact(emu):
    """Inputs filled with the rank: the sum must be n(n-1)/2 exactly (test/collectives_all.lua:298-304)."""
    from torchmpi_b200._lib import lib, check
    h, W = emu, emu.world
    lib.tmpi_cuda_heap_reset_allocator(0)
    n = 70000 // (4 * W) * (4 * W)
    off, ts = fill(h, n, torch.float32, 0)
    for r, t in enumerate(ts):
        t.fill_(float(r))
    g, keep = group(W)
    for algo in (2, 1 if n * 4 <= (512 << 10) else 2):
        for r, t in enumerate(ts):
            t.fill_(float(r))
        check(lib.tmpi_cuda_allreduce_heap(off, off, n, 7, 1.0, C.byref(g), algo, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        for t in ts:
            assert torch.all(t == W * (W - 1) / 2)
    status_ok(h)


def test_oneshot_slots_stay_inside_their_lane(emu):
    """One-shot allreduces on lane 0 and lane 1, even and odd epochs: each lane may only write its own
    2 * world slots; the other lanes' slots and the bounce buffers must keep their contents."""
    from torchmpi_b200._lib import lib, check
    h, W = emu, emu.world
    lib.tmpi_cuda_heap_reset_allocator(0)
    lay = h.layout()
    n = 4096
    off, ts = fill(h, n, torch.float32, 21)
    want = sum(t.double() for t in ts)
    region = lay["arena_off"] - lay["slots_off"]               # slots of all lanes + both bounce buffers
    lane_bytes = 2 * W * lay["slot_bytes"]
    views = [h.view(lay["slots_off"], region, peer=r) for r in range(W)]
    for lane in (0, 1):
        for v in views:
            v.fill_(0x5A)
        g, keep = group(W, lane)
        for _ in range(3):                                      # consecutive epochs: both parities are used
            for r, t in enumerate(ts):
                t.copy_(torch.randn(n, generator=torch.Generator(device="cuda").manual_seed(21 + r), device="cuda"))
            want = sum(t.double() for t in ts)
            check(lib.tmpi_cuda_allreduce_heap(off, off, n, 7, 1.0, C.byref(g), 1, torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            h.check_status(lane)
            for t in ts:
                assert torch.allclose(t.double(), want, atol=1e-4)
        lo, hi = lane * lane_bytes, (lane + 1) * lane_bytes
        for v in views:
            assert bool((v[:lo] == 0x5A).all()) and bool((v[hi:] == 0x5A).all()), f"lane {lane} wrote outside its slots"
            assert not bool((v[lo:hi] == 0x5A).all())


@pytest.mark.parametrize("algo", [1, 2, 5])    # 1 = pull (auto small), 2 = chunked, 5 = scatter + push in one pass
def test_broadcast(emu, algo):
    from torchmpi_b200._lib import lib, check
    h, W = emu, emu.world
    lib.tmpi_cuda_heap_reset_allocator(0)
    for n in (16, 4099 * 16, 1 << 20):
        for root in (W - 1, 0):
            off, ts = fill(h, n, torch.uint8 if False else torch.int8, 3)
            want = ts[root].clone()
            g, keep = group(W)
            check(lib.tmpi_cuda_broadcast_heap(off, n, 1, root, C.byref(g), algo, torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            status_ok(h)
            for t in ts:
                assert torch.equal(t, want)


def test_reduce_allgather_reduce_scatter(emu):
    from torchmpi_b200._lib import lib, check
    h, W = emu, emu.world
    lib.tmpi_cuda_heap_reset_allocator(0)
    s = torch.cuda.current_stream().cuda_stream
    n = 8192
    in_off, ins = fill(h, n, torch.float32, 5)
    out_off, outs = fill(h, n, torch.float32, 6)
    before = [o.clone() for o in outs]
    g, keep = group(W)
    root = 1 % W
    check(lib.tmpi_cuda_reduce(in_off, out_off, n, 7, root, C.byref(g), s))   # emulation: pointers are offsets
    torch.cuda.synchronize()
    ref = sum(t.double() for t in ins)
    for r in range(W):
        if r == root:
            assert torch.allclose(outs[r].double(), ref, atol=1e-4)
        else:
            assert torch.equal(outs[r], before[r])
    # allgather: rank r contributes n_r = 256 * (r + 1) floats
    counts = [256 * (r + 1) for r in range(W)]
    in_off, ins = fill(h, max(counts), torch.float32, 7)
    total = sum(counts)
    out_off, outs = fill(h, total, torch.float32, 8)
    carr = (C.c_int64 * W)(*counts)
    check(lib.tmpi_cuda_allgatherv(in_off, out_off, counts[0], carr, 7, C.byref(g), s))
    torch.cuda.synchronize()
    want = torch.cat([ins[r][:counts[r]] for r in range(W)])
    for r in range(W):
        assert torch.equal(outs[r], want)
    # reduce_scatter: n_out per rank
    n_out = 4096
    in_off, ins = fill(h, n_out * W, torch.bfloat16, 9)
    out_off, outs = fill(h, n_out, torch.bfloat16, 10)
    check(lib.tmpi_cuda_reduce_scatter(in_off, out_off, n_out, 6, 1.0, C.byref(g), s))
    torch.cuda.synchronize()
    ref = sum(t.double() for t in ins)
    for r in range(W):
        assert torch.allclose(outs[r].double(), ref[r * n_out:(r + 1) * n_out], atol=0.08 * W ** 0.5, rtol=0.02)
    check(lib.tmpi_cuda_barrier(C.byref(g), s))
    torch.cuda.synchronize()
    status_ok(h)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_allreduce_sgd_matches_torch_sgd(emu, dtype):
    """Three steps of the fused kernel against torch.optim.SGD fed with the summed gradients."""
    from torchmpi_b200._lib import lib, check, SgdBucket
    h, W = emu, emu.world
    lib.tmpi_cuda_heap_reset_allocator(0)
    n = 128 * W * 37
    shard = n // W
    g_off, grads = fill(h, n, dtype, 11)
    w_off, weights = fill(h, n, dtype, 12)
    for wt in weights[1:]:
        wt.copy_(weights[0])
    lr, mom, wd, scale = 0.1, 0.9, 1e-4, 1.0 / W
    ref_w = torch.nn.Parameter(weights[0].float().clone())
    opt = torch.optim.SGD([ref_w], lr=lr, momentum=mom, weight_decay=wd, nesterov=True)
    use_master = dtype != torch.float32
    master = weights[0].float().clone() if use_master else None           # all shards back to back
    momentum = torch.zeros(n, dtype=torch.float32, device="cuda")
    gr, keep = group(W, lane=2)
    for step in range(3):
        gen = torch.Generator(device="cuda").manual_seed(100 + step)
        for r in range(W):
            grads[r].copy_(torch.randn(n, generator=gen, device="cuda").to(dtype))
        ref_w.grad = sum(t.float() for t in grads) * scale
        opt.step()
        b = SgdBucket()
        b.grad_off, b.weight_off, b.n = g_off, w_off, n
        b.master = master.data_ptr() if use_master else None
        b.momentum = momentum.data_ptr()
        b.grad_dtype = b.weight_dtype = DT[dtype]
        b.lr, b.momentum_coef, b.dampening, b.weight_decay, b.grad_scale = lr, mom, 0.0, wd, scale
        b.nesterov, b.first_step, b.zero_grads = 1, int(step == 0), 1
        check(lib.tmpi_cuda_allreduce_sgd(C.byref(b), C.byref(gr), 2, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        h.check_status(2)
        for r in range(W):
            assert torch.equal(weights[r], weights[0]), "replicas must receive identical weights"
            assert torch.count_nonzero(grads[r]) == 0, "gradients must be cleared"
        got = master if use_master else weights[0]
        assert torch.allclose(got, ref_w.detach(), atol=2e-5, rtol=1e-5), (step, (got - ref_w).abs().max())
        if use_master:
            assert torch.equal(weights[0], master.to(dtype))
    assert shard * W == n


def test_bounded_wait_reports_timeout_and_context_survives(emu):
    """A wait on a flag nobody sets must give up after its budget, report status 3 and leave the
    context usable (no trap, no hang)."""
    from torchmpi_b200._lib import lib
    import time
    t0 = time.time()
    code = lib.tmpi_cuda_test_wait_timeout(300, torch.cuda.current_stream().cuda_stream)
    dt = time.time() - t0
    assert code == 3
    assert 0.25 < dt < 5.0
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0
