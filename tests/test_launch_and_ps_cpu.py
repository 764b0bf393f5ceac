"""Launcher, CPU parameter server scenarios and the Update schedules (no GPU)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

from mp_util import run_ranks

ENV = dict(os.environ, PYTHONPATH=str(Path(__file__).resolve().parent.parent))


def test_launcher_runs_ranks_and_reports_failure(tmp_path):
    ok = tmp_path / "ok.py"
    ok.write_text(textwrap.dedent("""
        import os, torchmpi_b200 as mpi
        mpi.start(with_cuda=False)
        assert mpi.size() == int(os.environ["WORLD_SIZE"]) == 2
        v = mpi.allreduce_int(mpi.rank() + 1)
        mpi.stop()
        if os.environ["RANK"] == "0":
            print("SUM", v)
    """))
    r = subprocess.run([sys.executable, "-m", "torchmpi_b200.launch", "--nproc", "2", str(ok)],
                       capture_output=True, text=True, timeout=120, env=ENV)
    assert r.returncode == 0, r.stderr
    assert "SUM 3" in r.stdout
    bad = tmp_path / "bad.py"
    bad.write_text("import os, sys, time\nif os.environ['RANK'] == '1':\n    print('boom'); sys.exit(7)\ntime.sleep(30)\n")
    r = subprocess.run([sys.executable, "-m", "torchmpi_b200.launch", "--nproc", "2", str(bad)],
                       capture_output=True, text=True, timeout=60, env=ENV)
    assert r.returncode == 7
    assert "rank 1 failed" in r.stderr and "boom" in r.stderr


def test_core_slices_partition_the_cores():
    from torchmpi_b200.launch import core_slice
    cores = list(range(16))
    got = [core_slice(r, 4, cores) for r in range(4)]
    assert got == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11], [12, 13, 14, 15]]


def _ps_scenarios(rank, world):
    """The five scenarios of test/parameterserver.lua on CPU tensors, plus DSGD == allreduce."""
    import torchmpi_b200 as mpi
    from torchmpi_b200 import parameterserver as ps
    mpi.start(with_cuda=False)
    n = world
    for dtype in (torch.float32, torch.float64):
        for it in range(10):
            t = torch.full((1000,), float(rank), dtype=dtype)
            server = ps.init(t)
            out = torch.empty_like(t)
            mpi.sync_handle(ps.receive(server, out))
            for r in range(n):
                b, e = ps.shard_range(1000, n, r)
                assert torch.all(out[b:e] == r)
            ps.free(server)
            t2 = torch.full((911, 101), float(rank), dtype=dtype)
            server = ps.init(t2)
            if rank == n - 1:
                mpi.sync_handle(ps.send(server, t2, "zero"))
            mpi.barrier()
            out2 = torch.empty_like(t2)
            mpi.sync_handle(ps.receive(server, out2))
            assert torch.all(out2 == 0)
            mpi.barrier()
            if rank == n - 1:
                mpi.sync_handle(ps.send(server, t2, "copy"))
            mpi.barrier()
            mpi.sync_handle(ps.receive(server, out2))
            assert torch.all(out2 == n - 1)
            mpi.barrier()
            mpi.sync_handle(ps.send(server, t2, "add"))
            mpi.barrier()
            mpi.sync_handle(ps.receive(server, out2))
            assert torch.all(out2 == n - 1 + n * (n - 1) / 2)
            ps.free(server)
    with pytest.raises(ValueError):
        ps.send(ps.init(torch.zeros(16)), torch.zeros(16), "none")      # the reference's default rule name asserts
    # parameter server as a synchronous allreduce (mnist_parameterserver_dsgd.lua:62-88)
    torch.manual_seed(rank)
    x = torch.randn(10007)
    ref = x.clone()
    mpi.gloo.allreduce_tensor(ref)
    server = ps.init(x)
    if rank == 0:
        mpi.sync_handle(ps.send(server, x, "zero"))
    mpi.barrier()
    mpi.sync_handle(ps.send(server, x, "add"))
    mpi.barrier()
    got = torch.empty_like(x)
    mpi.sync_handle(ps.receive(server, got))
    assert torch.allclose(got, ref, atol=1e-5)
    ps.free_all()
    mpi.stop()
    return True


def _ps_serialized(rank, world):
    """Every rank overwrites the whole server with its own value, all at once and without barriers: with
    ``serialized=True`` the server always holds one rank's complete message (lib/parameterserver.cpp:426-499 applies
    one message at a time per shard), so after the last round every shard holds the same client's value, and the adds
    that follow are all counted."""
    import torchmpi_b200 as mpi
    from torchmpi_b200 import parameterserver as ps
    mpi.start(with_cuda=False)
    n = world
    server = ps.init(torch.zeros(40_000))
    out = torch.empty(40_000)
    for it in range(8):
        h = ps.send(server, torch.full((40_000,), float(rank + 1 + 10 * it)), "copy", serialized=True)
        assert h.done()                 # the update is in place when the call returns
    mpi.barrier()
    mpi.sync_handle(ps.receive(server, out))
    winner = float(out[0])
    assert torch.all(out == winner) and winner in [float(r + 1 + 70) for r in range(n)]
    mpi.barrier()
    ps.send(server, torch.ones(40_000), "add", serialized=True)
    mpi.barrier()
    mpi.sync_handle(ps.receive(server, out))
    assert torch.all(out == winner + n)
    ps.free_all()
    mpi.stop()
    return True


def test_cpu_parameter_server_serialized_sends():
    assert all(run_ranks(_ps_serialized, 4, timeout=300))


def test_cpu_parameter_server_scenarios():
    assert all(run_ranks(_ps_scenarios, 4, timeout=300))


def _policies(rank, world):
    """Downpour and EASGD schedules on a small model, with a data-parallel level under the sharding level."""
    import torchmpi_b200 as mpi
    from torchmpi_b200 import parameterserver as ps
    from torchmpi_b200 import nn as mpinn

    def groups():
        return mpi.push_communicator(str(mpi.rank() // 2))

    mpi.start(with_cuda=False, custom_communicator_init=groups)
    mpi.set_communicator(0)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(20, 30), torch.nn.ReLU(), torch.nn.Linear(30, 5))
    # EASGD across everybody (sharding and data-parallel communicator both 0)
    upd = ps.EASGDUpdate(net, 0, 0, beta=0.8, update_frequency=4, init_delay=2, prefetch=1)
    assert (upd.next_integration, upd.next_prefetch, upd.next_send) == (6, 7, 6)
    events = []
    start = [p.detach().clone() for p in net.parameters()]
    for step in range(1, 20):
        with torch.no_grad():
            for p in net.parameters():
                p.add_(0.01 * (rank + 1))               # ranks drift apart
        before = [p.detach().clone() for p in net.parameters()]
        upd.update(step)
        moved = any(not torch.equal(a, b) for a, b in zip(before, net.parameters()))
        if moved:
            events.append(step)
    assert events == [6, 10, 14, 18], events           # init_delay + k * update_frequency
    assert mpi.communicator_level() == 0
    # the centre has moved towards the mean drift; pull it and compare with a replay of the elastic rule
    ps.sync_handles(upd.handles_send)
    mpi.barrier()
    centre = [torch.empty_like(p) for p in net.parameters()]
    hs = [ps.receive(ps.cache.parameter_servers[ps.cache.key(p.data)][1], c) for p, c in zip(net.parameters(), centre)]
    ps.sync_handles(hs)
    for c, s0 in zip(centre, start):
        assert torch.isfinite(c).all() and not torch.equal(c, s0)
    mpinn.check_with_allreduce(centre)                  # every rank sees the same centre
    ps.free_all()
    # Downpour with a separate data-parallel level: only group roots talk to the server
    net2 = torch.nn.Linear(16, 16)
    mpi.set_collective_span(1, 1)
    mpinn.synchronize_parameters(net2)
    mpi.set_collective_span(0, 0)
    d = ps.DownpourUpdate(net2, 0, 1, update_frequency=3, init_delay=1, prefetch=0, send_frequency=2,
                          local_update=lambda t: t.mul_(-0.1))
    assert d.next_send == 3 and d.next_integration == 4
    for step in range(1, 12):
        for p in net2.parameters():
            p.grad = torch.full_like(p, 1.0)
        d.update(step)
    mpi.set_communicator(1)
    mpinn.check_with_allreduce(net2)                    # group members agree after the broadcasts
    mpi.set_communicator(0)
    ps.free_all()
    mpi.stop()
    return True


def test_update_policies_schedule():
    assert all(run_ranks(_policies, 4, timeout=300))
