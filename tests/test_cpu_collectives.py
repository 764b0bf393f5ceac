"""CPU ranks (gloo control plane + shared-memory heap): start/stop, communicators, the collective matrix.

Modelled on test/startstop.lua, test/hierarchical_communicators.lua and the correctness half of
test/collectives_all.lua: inputs are filled with the rank, so an allreduce over n ranks must give
n(n-1)/2 exactly, a broadcast from the last rank n-1, and so on.
"""
import pytest
import torch

from mp_util import run_ranks

DTYPES = [torch.int8, torch.int32, torch.int64, torch.float32, torch.float64, torch.bfloat16]
SIZES = [1, 7, 256, 4099, 1 << 16]


def _startstop(rank, world):
    import torchmpi_b200 as mpi
    mpi.start(with_cuda=False)
    assert mpi.rank() == rank and mpi.size() == world
    names = mpi.communicator_names()
    assert "key(global)" in names
    assert mpi.num_communicators == 2          # global + per-node level
    assert mpi.collective_span() == (0, 1)
    assert not mpi.need_inter_node_collectives
    mpi.barrier()
    avail = mpi.collective_availability()
    assert "MPI.p2p.allreduceTensor" in avail and "cpu = {" in avail
    sel = mpi.collective_selector_to_string("cpu", "singlenode", "sync")
    assert "cpu.singlenode.sync.allreduceTensor" in sel
    mpi.stop()
    return True


@pytest.mark.parametrize("world", [1, 3])
def test_start_stop(world):
    assert all(run_ranks(_startstop, world))


def _hierarchy(rank, world):
    import torchmpi_b200 as mpi
    div = 3

    def custom():
        lvl = mpi.C.torchmpi_push_communicator(str(mpi.rank() % div))
        assert lvl == 1
        return lvl

    mpi.start(with_cuda=False, with_ipc_groups=False, custom_communicator_init=custom,
              with_cartesian_communicator=True)
    mpi.set_communicator(0)
    assert mpi.is_cartesian_communicator()
    assert mpi.size() == world
    rank_g = mpi.rank()
    mpi.set_communicator(1)
    rank_l1, size_l1 = mpi.rank(), mpi.size()
    cart = world < div or world % div == 0
    assert cart or not mpi.is_cartesian_communicator()
    assert rank_g // div == rank_l1
    # scalar collectives act on the communicator under the cursor
    assert mpi.allreduce_int(1) == size_l1
    assert mpi.broadcast_double(0, float(rank_g)) == float(rank_g % div)   # group root has global rank r % div
    mpi.set_communicator(2)          # per-node level: everyone of level 1 is on this host
    assert mpi.size() == size_l1
    mpi.set_communicator(0)
    assert mpi.allreduce_long(rank_g) == world * (world - 1) // 2
    assert mpi.reduce_double(0, 2.0) == (2.0 * world if rank_g == 0 else 2.0)
    assert mpi.sendreceive_int(rank_g, (rank_g - 1) % world, (rank_g + 1) % world) == (rank_g - 1) % world
    mpi.barrier()
    mpi.stop()
    return True


@pytest.mark.parametrize("world", [4, 6])
def test_hierarchical_communicators(world):
    assert all(run_ranks(_hierarchy, world))


def _matrix(rank, world):
    import torchmpi_b200 as mpi
    mpi.start(with_cuda=False)
    assert mpi._S.shm_ready, "host heap should be available for ranks of one host"
    n = world
    for backend_ns, name in ((mpi, "selector"), (mpi.p2p, "p2p"), (mpi.gloo, "gloo")):
        for dt in DTYPES:
            if name == "gloo" and dt == torch.bfloat16:
                continue
            for size in SIZES:
                # allreduce in place
                t = torch.full((size,), rank, dtype=dt)
                backend_ns.allreduce_tensor(t)
                assert torch.all(t == n * (n - 1) // 2), (name, dt, size, t[:4])
                # allreduce out of place leaves the input untouched
                inp, out = torch.full((size,), rank, dtype=dt), torch.full((size,), -1, dtype=dt)
                backend_ns.allreduce_tensor(inp, out)
                assert torch.all(inp == rank) and torch.all(out == n * (n - 1) // 2)
                # broadcast from the last rank
                t = torch.full((size,), rank, dtype=dt)
                backend_ns.broadcast_tensor(n - 1, t)
                assert torch.all(t == n - 1)
    # every p2p algorithm gives the same bits on every rank for float data
    torch.manual_seed(1234 + rank)
    for algo in ("oneshot", "twoshot", "ring"):
        x = torch.randn(70001)
        ref = x.clone()
        mpi.gloo.allreduce_tensor(ref)
        y = x.clone()
        mpi.p2p.allreduce_tensor(y, algo=algo, scale=0.5)
        assert torch.allclose(y, ref * 0.5, rtol=1e-5, atol=1e-5), algo
        mpi.check_with_allreduce(y, f"replicated result of {algo}")
    # reduce: only the root's output changes
    for ns in (mpi, mpi.p2p):
        for size in SIZES:
            inp, out = torch.full((size,), float(rank)), torch.full((size,), -1.0)
            ns.reduce_tensor(0, inp, out)
            assert torch.all(inp == rank)
            assert torch.all(out == (n * (n - 1) / 2 if rank == 0 else -1.0))
    # sendreceive: ring shift
    t = torch.full((1000,), float(rank))
    mpi.sendreceive_tensor(t, (rank - 1) % n, (rank + 1) % n)
    assert torch.all(t == (rank - 1) % n)
    # allgather with per-rank sizes and an undersized output (auto resize)
    for ns in (mpi, mpi.p2p):
        inp = torch.full((5 + rank,), float(rank))
        out = torch.empty(1)
        res = ns.allgather_tensor(inp, out)
        expect = torch.cat([torch.full((5 + r,), float(r)) for r in range(n)])
        assert res.numel() == expect.numel() and torch.equal(res.view(-1), expect)
    # equal contributions announced by the caller: no count exchange on the control plane
    for ns in (mpi, mpi.p2p):
        res = ns.allgather_tensor(torch.full((7,), float(rank)), torch.empty(7 * n), equal_counts=True)
        assert torch.equal(res.view(-1), torch.arange(n, dtype=torch.float32).repeat_interleave(7))
    # reduce_scatter
    inp = torch.arange(n * 10, dtype=torch.float32) + rank
    out = torch.empty(10)
    mpi.reduce_scatter_tensor(inp, out)
    base = torch.arange(rank * 10, rank * 10 + 10, dtype=torch.float32)
    assert torch.equal(out, base * n + n * (n - 1) / 2)
    # async flavours return handles; the launch itself must be quick
    import time
    for ns in (mpi.async_, mpi.async_.p2p, mpi.async_.gloo):
        t = torch.full((1 << 16,), float(rank))
        t0 = time.perf_counter()
        h = ns.allreduce_tensor(t)
        launch_us = (time.perf_counter() - t0) * 1e6
        mpi.sync_handle(h)
        assert torch.all(t == n * (n - 1) / 2)
        assert launch_us < 50000
        t = torch.full((4097,), float(rank))
        h = ns.broadcast_tensor(0, t)
        mpi.sync_handle(h)
        assert torch.all(t == 0)
    # non-contiguous tensors are rejected
    with pytest.raises(ValueError):
        mpi.allreduce_tensor(torch.zeros(4, 4).t())
    mpi.barrier()
    mpi.stop()
    return True


@pytest.mark.parametrize("world", [2, 3, 5, 8])
def test_collective_matrix(world):
    assert all(run_ranks(_matrix, world, timeout=300))


def _hier_allreduce(rank, world, cartesian):
    import torchmpi_b200 as mpi

    def custom():
        return mpi.push_communicator(str(mpi.rank() // 2))     # groups of 2

    if True:
        mpi.start(with_cuda=False, custom_communicator_init=custom, with_cartesian_communicator=cartesian)
        mpi.set_collective_span(0, 1)          # outer = everyone, inner = the groups of 2
        assert mpi.is_cartesian_communicator(1) == cartesian
        t = torch.full((5000,), float(rank))
        mpi.allreduce_tensor(t)
        assert torch.all(t == world * (world - 1) / 2), (cartesian, t[:3])
        mpi.config.set_flat_collectives()
        t = torch.full((5000,), float(rank))
        mpi.allreduce_tensor(t)
        assert torch.all(t == world * (world - 1) / 2)
        mpi.config.set_hierarchical_collectives()
        # asynchronous flavour on the hierarchical span: a live handle at once, the whole chain behind it
        import time
        t = torch.full((5000,), float(rank))
        t0 = time.perf_counter()
        h = mpi.async_.allreduce_tensor(t)
        launch_us = (time.perf_counter() - t0) * 1e6
        assert h is not None and launch_us < 50000
        mpi.sync_handle(h)
        assert torch.all(t == world * (world - 1) / 2), (cartesian, t[:3])
        # reduce to a root that is not the first member of its group
        for root in range(world):
            src = torch.full((777,), float(rank + 1))
            dst = torch.full((777,), -1.0)
            mpi.reduce_tensor(root, src, dst)
            assert torch.all(src == rank + 1)
            if rank == root:
                assert torch.all(dst == world * (world + 1) / 2), (cartesian, root, dst[:3])
            else:
                assert torch.all(dst == -1.0)
        mpi.stop()
    return True


@pytest.mark.parametrize("cartesian", [True, False])
def test_hierarchical_allreduce_equals_flat(cartesian):
    assert all(run_ranks(_hier_allreduce, 4, cartesian))


def _independent_push(rank, world):
    """Two disjoint groups of a level split themselves independently: only the members of a communicator take
    part in its push (lib/c_api.h:42-47), so one group can push a level the other never does."""
    import torchmpi_b200 as mpi
    mpi.start(with_cuda=False)
    base = mpi.num_communicators
    lvl1 = mpi.push_communicator("left" if rank < 2 else "right")          # {0, 1} and {2, 3}
    assert mpi.size() == 2
    if rank < 2:
        # only the left group goes deeper, twice, while the right group works at its own level
        lvl2 = mpi.push_communicator(f"solo{rank}")
        assert mpi.size() == 1 and lvl2 == lvl1 + 1
        mpi.set_communicator(lvl1)
        lvl3 = mpi.push_communicator("again")
        assert mpi.size() == 2 and lvl3 == lvl2 + 1
        t = torch.full((100,), float(rank))
        mpi.set_collective_span(lvl3, lvl3)
        mpi.allreduce_tensor(t)
        assert torch.all(t == 1.0)
        assert mpi.num_communicators == base + 3
    else:
        t = torch.full((100,), float(rank))
        mpi.set_collective_span(lvl1, lvl1)
        for _ in range(3):
            mpi.allreduce_tensor(t, scale=0.5)
        assert torch.all(t == 2.5)
        assert mpi.num_communicators == base + 1
        assert mpi.num_nodes_in_communicator() == 1
    mpi.set_communicator(0)
    mpi.barrier()
    mpi.stop()
    return True


def test_groups_push_communicators_independently():
    assert all(run_ranks(_independent_push, 4))
