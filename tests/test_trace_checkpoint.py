"""Tracing ring buffer and checkpoint/resume among CPU ranks."""
import os

import torch

from mp_util import run_ranks


def _trace_and_checkpoint(rank, world, tmpdir):
    import torchmpi_b200 as mpi
    from torchmpi_b200.utils import trace, checkpoint
    from torchmpi_b200.models.mlp import MLP
    mpi.start(with_cuda=False)
    trace.clear()
    trace.enable()
    t = torch.ones(1000)
    mpi.allreduce_tensor(t)
    mpi.broadcast_tensor(0, t)
    with trace.range("user region"):
        pass
    rows = trace.records()
    trace.enable(False)
    assert [r["op"] for r in rows] == ["allreduce", "broadcast"]
    assert rows[0]["bytes"] == 4000 and rows[0]["us"] > 0
    n = trace.dump(os.path.join(tmpdir, f"trace_{rank}.jsonl"))
    assert n == 2
    mpi.allreduce_tensor(t)
    assert len(trace.records()) == 2          # disabled: nothing more recorded
    # checkpoint: rank 0's model is saved; a differently initialised model resumes to the same bits everywhere
    torch.manual_seed(rank)
    model = MLP()
    from torchmpi_b200 import nn as mpinn
    mpinn.synchronize_parameters(model)
    path = os.path.join(tmpdir, "ckpt.pt")
    checkpoint.save(path, model, extra={"step": 7})
    want = [p.detach().clone() for p in model.parameters()]
    torch.manual_seed(100 + rank)
    other = MLP()
    extra = checkpoint.load(path, other)
    assert extra == {"step": 7}
    for a, b in zip(other.parameters(), want):
        assert torch.equal(a, b)
    mpinn.check_with_allreduce(other)
    # parameter-server shards travel with the checkpoint: what the servers hold at save time is what they hold after load
    from torchmpi_b200 import parameterserver as ps
    seed = torch.arange(1000, dtype=torch.float32) * (1.0 if rank == 0 else 0.0)
    server = ps.init(seed.clone())
    if rank == 0:
        ps.send(server, torch.arange(1000, dtype=torch.float32) + 5.0, "copy").wait()
    mpi.barrier()
    path2 = os.path.join(tmpdir, "ckpt_ps.pt")
    checkpoint.save(path2, model, parameter_servers=[server])
    if rank == 0:
        ps.send(server, torch.zeros(1000), "zero").wait()       # lose the contents
    mpi.barrier()
    checkpoint.load(path2, other, parameter_servers=[server])
    got = torch.empty(1000)
    ps.receive(server, got).wait()
    assert torch.equal(got, torch.arange(1000, dtype=torch.float32) + 5.0)
    mpi.stop()
    return True


def test_trace_and_checkpoint(tmp_path):
    assert all(run_ranks(_trace_and_checkpoint, 2, str(tmp_path)))
