"""Failure detection among CPU ranks: every failure is made on the host (a rank that exits between steps, a
rank whose heartbeat stalls, a parameter-server request that is dropped); the survivors must get a clean
error within the budget instead of waiting for ever, and later calls must fail at once (poisoning)."""
import os
import time

import pytest
import torch

from mp_util import run_ranks


def _common(budget_ms=1500, interval_ms=100):
    import torchmpi_b200 as mpi
    from torchmpi_b200 import config
    config.set("watchdog_interval_ms", interval_ms)
    config.set("watchdog_budget_ms", budget_ms)
    mpi.start(with_cuda=False)
    return mpi


def _rank_exits(rank, world):
    mpi = _common()
    t = torch.ones(100)
    mpi.allreduce_tensor(t)                 # a healthy step
    assert torch.all(t == world)
    mpi.barrier()
    if rank == world - 1:
        return -1.0                         # leaves between steps: no stop(), no goodbye, nothing in flight; the process ends
    t0 = time.time()
    while mpi.watchdog.poisoned() is None and time.time() - t0 < 20:
        time.sleep(0.05)
    took = time.time() - t0
    assert mpi.watchdog.poisoned() is not None and f"rank {world - 1}" in mpi.watchdog.poisoned(), mpi.watchdog.poisoned()
    assert took < 10, took
    t1 = time.time()
    with pytest.raises(mpi.CommunicatorPoisoned):
        mpi.allreduce_tensor(t)             # fails at once, does not wait for the lost rank
    with pytest.raises(mpi.CommunicatorPoisoned):
        mpi.barrier()
    assert time.time() - t1 < 1.0
    mpi.stop()                              # teardown still works (no barrier with a lost peer)
    return took


def test_rank_that_exits_between_steps_is_detected():
    world = 3
    res = run_ranks(_rank_exits, world, timeout=120)
    assert res[world - 1] == -1.0 and all(0 <= r < 10 for r in res[:world - 1]), res


def _rank_stalls(rank, world):
    mpi = _common()
    mpi.barrier()
    if rank == 1:
        mpi.watchdog.pause(True)            # the host thread of this rank stops answering (a stall), the process lives
        time.sleep(4.0)
        mpi.watchdog.pause(False)
        mpi.watchdog.poison("the peers have given up on this rank meanwhile")   # so that stop() does not wait for them
        mpi.stop()
        return "stalled"
    t0 = time.time()
    while mpi.watchdog.poisoned() is None and time.time() - t0 < 20:
        time.sleep(0.05)
    reason = mpi.watchdog.poisoned()
    assert reason is not None and "rank 1" in reason, reason
    assert time.time() - t0 < 4.0           # within the budget (1.5 s) plus slack, before the stall even ends
    with pytest.raises(mpi.CommunicatorPoisoned):
        mpi.allreduce_tensor(torch.ones(4))
    mpi.stop()
    return "detected"


def test_rank_that_stalls_past_the_budget_is_detected():
    res = run_ranks(_rank_stalls, 2, timeout=120)
    assert res == ["detected", "stalled"]


def _dropped_request(rank, world):
    mpi = _common(budget_ms=60000)
    from torchmpi_b200 import config, parameterserver as ps
    server = ps.init(torch.zeros(1000))
    mpi.barrier()
    outcome = "ok"
    if rank == 0:
        config.set("fault_drop_ps_requests", 1)      # the next request is lost on the way
        h = ps.send(server, torch.ones(1000), "add")
        t0 = time.time()
        with pytest.raises(mpi.TimeoutError):
            h.wait(timeout_ms=500)
        assert time.time() - t0 < 3.0
        config.set("fault_drop_ps_requests", 0)
        with pytest.raises(mpi.CommunicatorPoisoned):   # the job is poisoned: nothing waits on this server again
            mpi.allreduce_tensor(torch.ones(4))
        outcome = "timeout"
    mpi.stop()
    return outcome


def test_dropped_parameter_server_request_times_out_cleanly():
    res = run_ranks(_dropped_request, 2, timeout=120)
    assert res[0] == "timeout"
