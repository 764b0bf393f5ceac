"""Checkpoint and resume.

The reference has no save / load at all (parameter-server shards live in host memory and vanish at
``free``, lib/parameterserver.cpp:277-280).  Here a checkpoint is a plain PyTorch file written by
rank 0: the model's ``state_dict`` (parameters are replicated, so rank 0's copy is the model), and,
when the fused optimizer is in use, its gathered fp32 master weights and momentum, and, when parameter
servers are passed, the tensors they hold (pulled from their shards before the file is written).  ``load``
restores them on every rank, re-synchronises the parameters from rank 0 and writes the saved tensors
back into the parameter servers.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import runtime
from ..runtime import S


def save(path: str, model: torch.nn.Module, optimizer=None, extra: Optional[dict] = None,
         parameter_servers: Optional[Sequence] = None) -> None:
    """Collective: every rank calls (the optimizer state is gathered, the parameter-server shards are pulled);
    rank 0 writes the file.  ``parameter_servers``: ``ParameterServer`` objects in an order that is the same
    at save and load."""
    state = {"model": {k: v.detach().cpu() for k, v in model.state_dict().items()}, "extra": extra or {}}
    if optimizer is not None and hasattr(optimizer, "state_dict"):
        state["optimizer"] = optimizer.state_dict()
    if parameter_servers:
        held = []
        for ps in parameter_servers:
            t = torch.empty(ps.n, dtype=ps.dtype, device=S.device if ps.on_gpu else "cpu")
            ps.receive(t).wait()
            held.append(t.cpu())
        state["parameter_servers"] = held
    if not S.started or S.rank == 0:
        torch.save(state, path)
    if S.started:
        runtime.barrier()


def load(path: str, model: torch.nn.Module, optimizer=None, synchronize: bool = True,
         parameter_servers: Optional[Sequence] = None) -> dict:
    """Every rank reads the file; parameters are then broadcast from rank 0 so that replicas hold the
    same bits even if the file systems differ."""
    state = torch.load(path, map_location="cpu", weights_only=False)
    with torch.no_grad():
        own = model.state_dict()
        for k, v in state["model"].items():
            if k in own:
                own[k].copy_(v.to(own[k].device, own[k].dtype))     # in place: flat-bucket views stay intact
    if synchronize and S.started and len(runtime.intra_members(runtime.collective_span()[0])) > 1:
        from .. import nn as mpinn
        mpinn.synchronize_parameters(model)
    if optimizer is not None and "optimizer" in state and hasattr(optimizer, "load_state_dict"):
        optimizer.load_state_dict(state["optimizer"])
        if hasattr(optimizer, "refresh_master") and state["optimizer"]["buckets"] and \
                state["optimizer"]["buckets"][0].get("master") is None:
            optimizer.refresh_master()
    if parameter_servers and "parameter_servers" in state:
        if len(parameter_servers) != len(state["parameter_servers"]):
            raise ValueError("the checkpoint holds another number of parameter-server tensors")
        for ps, t in zip(parameter_servers, state["parameter_servers"]):
            if runtime.rank() == 0:          # one writer, rule `copy`, as parameterserver.init_tensors seeds them
                ps.send(t.to(S.device if ps.on_gpu else "cpu").contiguous(), "copy").wait()
        if S.started:
            runtime.barrier()
    return state.get("extra", {})
