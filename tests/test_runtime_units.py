"""In-process tests of the native host runtime: tunables, handles, pools, split, ring plan."""
import ctypes as C
import time

import pytest

from torchmpi_b200 import _lib, config
from torchmpi_b200._lib import lib

KEY = 1024


def push(world, rank, keyfn, parent=None):
    parent = list(range(world)) if parent is None else parent
    buf = bytearray(KEY * len(parent))
    for i, r in enumerate(parent):
        k = str(keyfn(r)).encode()
        buf[i * KEY:i * KEY + len(k)] = k
    lvl = lib.tmpi_comm_push(bytes(buf), _lib.int_array(parent), len(parent), str(keyfn(rank)).encode())
    assert lvl >= 0, _lib.last_error()
    return lvl


def members(level, inter):
    out = (C.c_int * 64)()
    n = lib.tmpi_comm_members(level, inter, out, 64)
    return [out[i] for i in range(n)]


def test_tunables_defaults_and_roundtrip():
    assert config.get("small_gpu_allreduce_size") == 1 << 16
    assert config.get("small_cpu_broadcast_size") == 1 << 13
    assert config.get("num_buffers_per_gpu_collective") == 3
    assert config.get("collective_num_threads") == 4
    assert config.get("parameterserver_num_threads") == 4
    # the collective in-flight limit has its own variable (the reference writes the PS one)
    old = config.get_collective_thread_pool_size()
    config.set_collective_thread_pool_size(1234)
    assert config.get_collective_thread_pool_size() == 1234
    assert config.get_parameterserver_thread_pool_size() == 1 << 20
    config.set_collective_thread_pool_size(old)
    with pytest.raises(_lib.TorchMPIError):
        config.set("no_such_knob", 1)
    config.set_flat_collectives()
    assert config.get("use_hierarchical_collectives") == 0
    config.set_hierarchical_collectives()
    assert config.get("use_hierarchical_collectives") == 1


def test_handles_and_pools():
    t0 = time.time()
    hs = [lib.tmpi_test_sleep_task(0, 50, 0) for _ in range(4)]
    assert time.time() - t0 < 0.04          # enqueue returns at once
    assert lib.tmpi_handle_done(hs[0]) in (0, 1)
    for h in hs:
        assert lib.tmpi_handle_wait(h, -1) == 0
    assert time.time() - t0 < 0.15          # 4 workers ran them side by side
    assert lib.tmpi_handle_wait(hs[0], -1) == 0   # a waited (unknown) id counts as complete
    h = lib.tmpi_test_sleep_task(1, 1, 3)
    assert lib.tmpi_handle_wait(h, -1) == 3       # the task's status comes back
    h = lib.tmpi_test_sleep_task(1, 300, 0)
    assert lib.tmpi_handle_wait(h, 20) == _lib.ERR_TIMEOUT  # bounded wait
    assert "still running" in _lib.last_error()
    assert lib.tmpi_handle_wait(h, -1) == 0
    assert lib.tmpi_sync_all() == 0
    assert lib.tmpi_handles_in_flight() == 0


@pytest.mark.parametrize("world", list(range(1, 38)))
def test_split_by_rank_mod_3(world):
    """The arithmetic of test/hierarchical_communicators.lua for 1..37 ranks."""
    div = 3
    for rank in range(world):
        lib.tmpi_set_tunable(b"use_cartesian_communicator", 1)
        assert lib.tmpi_comm_reset(rank, world) == 0
        assert lib.tmpi_comm_is_cartesian(0) == 1
        lvl = push(world, rank, lambda r: r % div)
        assert lvl == 1 and lib.tmpi_comm_level() == 1
        intra, inter = members(1, 0), members(1, 1)
        assert intra == [r for r in range(world) if r % div == rank % div]
        assert lib.tmpi_comm_rank_in(1, 0) == rank // div
        cart = world < div or world % div == 0
        assert bool(lib.tmpi_comm_is_cartesian(1)) == cart
        if cart:
            assert inter == [r for r in range(world) if r // div == rank // div]
        elif rank // div == 0:
            assert inter == [r for r in range(world) if r // div == 0]   # roots only
        else:
            assert inter == [rank]
        # a second level splits the level-1 intra group (the cursor) again
        nodes = 2
        lvl2 = push(world, rank, lambda r: (r // div) % nodes, parent=intra)
        assert lvl2 == 2
        assert lib.tmpi_comm_rank_in(2, 0) == (rank // div) // nodes
        assert lib.tmpi_comm_has_inter_collective(2) == (1 if len(members(2, 0)) != len(intra) else 0)
        assert lib.tmpi_comm_set(0) == 0
        assert lib.tmpi_comm_set(7) != 0     # out of range is an error, not silently accepted
    lib.tmpi_set_tunable(b"use_cartesian_communicator", 0)


def test_tree_communicator_and_span():
    lib.tmpi_set_tunable(b"use_cartesian_communicator", 0)
    lib.tmpi_comm_reset(5, 8)
    push(8, 5, lambda r: r // 4)
    assert members(1, 0) == [4, 5, 6, 7]
    assert lib.tmpi_comm_is_cartesian(1) == 0
    assert members(1, 1) == [5]               # not a root: singleton inter group
    lib.tmpi_comm_reset(4, 8)
    push(8, 4, lambda r: r // 4)
    assert members(1, 1) == [0, 4]            # roots are linked
    assert lib.tmpi_comm_set_span(0, 1) == 0
    b, e = C.c_int(), C.c_int()
    lib.tmpi_comm_get_span(C.byref(b), C.byref(e))
    assert (b.value, e.value) == (0, 1)
    assert lib.tmpi_comm_set_span(0, 5) != 0
    buf = C.create_string_buffer(4096)
    lib.tmpi_comm_names(buf, 4096)
    assert "key(global)" in buf.value.decode() and "cartesian: false" in buf.value.decode()


@pytest.mark.parametrize("size", [1, 2, 3, 4, 7, 8])
def test_ring_plan_covers_every_chunk(size):
    """After the reduce phase ring index (c-1) mod size owns chunk c; the broadcast phase spreads it."""
    chunks = size
    for phase in (0, 1):
        n = (size - 1) * chunks * 2
        out = (C.c_int * max(1, n))()
        assert lib.tmpi_ring_plan(chunks, size, phase, out, n) == n
        for s in range(size - 1):
            seen_send, seen_recv = set(), set()
            for c in range(chunks):
                snd, rcv = out[(s * chunks + c) * 2], out[(s * chunks + c) * 2 + 1]
                assert rcv == (snd + 1) % size           # always to the next ring index
                assert lib.tmpi_ring_send_chunk(snd, size, s, phase) == c
                assert lib.tmpi_ring_recv_chunk(rcv, size, s, phase) == c
                seen_send.add(snd), seen_recv.add(rcv)
            assert len(seen_send) == chunks and len(seen_recv) == chunks   # every rank busy each step
    # simulate: contributions[c] = set of ranks summed into chunk c held by its current owner
    if size > 1:
        held = {(i, c): {i} for i in range(size) for c in range(size)}
        for s in range(size - 1):
            new = dict(held)
            for i in range(size):
                c = lib.tmpi_ring_recv_chunk(i, size, s, 0)
                new[(i, c)] = held[(i, c)] | held[((i - 1) % size, c)]
            held = new
        for c in range(size):
            assert held[((c - 1) % size, c)] == set(range(size))


def test_shard_ranges():
    b, e = C.c_size_t(), C.c_size_t()
    n, size = 911 * 101, 4
    covered = 0
    for r in range(size):
        assert lib.tmpi_ps_shard_range(n, size, r, C.byref(b), C.byref(e)) == 0
        assert b.value == covered
        assert e.value - b.value == n // size + (1 if r < n % size else 0)
        covered = e.value
    assert covered == n


def test_linear_ops_fall_back_to_pytorch_on_cpu():
    """``ops.gemm`` wrappers (GELU, bias gradient, Linear) use PyTorch where the CUDA kernels do not apply."""
    import torch
    from torchmpi_b200.ops import gemm
    torch.manual_seed(0)
    z, dy = torch.randn(16, 64), torch.randn(16, 64)
    assert torch.allclose(gemm.gelu(z), torch.nn.functional.gelu(z))
    dz, db = gemm.bias_grad(dy, z)
    ref = torch.ops.aten.gelu_backward(dy, z)
    assert torch.allclose(dz, ref) and torch.allclose(db, ref.sum(0))
    same, db2 = gemm.bias_grad(dy)
    assert same is dy and torch.allclose(db2, dy.sum(0))
    lin = gemm.Linear(64, 32, gelu=True)
    x = torch.randn(4, 64, requires_grad=True)
    lin(x).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    torch.nn.functional.gelu(torch.nn.functional.linear(xr, lin.weight.detach(), lin.bias.detach())).sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-6)
