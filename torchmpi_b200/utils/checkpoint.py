"""Checkpoint and resume.

The reference has no save / load at all (parameter-server shards live in host memory and vanish at
``free``, lib/parameterserver.cpp:277-280).  Here a checkpoint is a plain PyTorch file written by
rank 0: the model's ``state_dict`` (parameters are replicated, so rank 0's copy is the model), and,
when the fused optimizer is in use, its gathered fp32 master weights and momentum.  ``load`` restores
them on every rank and re-synchronises the parameters from rank 0.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime
from ..runtime import S


def save(path: str, model: torch.nn.Module, optimizer=None, extra: Optional[dict] = None) -> None:
    """Collective: every rank calls (the optimizer state is gathered); rank 0 writes the file."""
    state = {"model": {k: v.detach().cpu() for k, v in model.state_dict().items()}, "extra": extra or {}}
    if optimizer is not None and hasattr(optimizer, "state_dict"):
        state["optimizer"] = optimizer.state_dict()
    if not S.started or S.rank == 0:
        torch.save(state, path)
    if S.started:
        runtime.barrier()


def load(path: str, model: torch.nn.Module, optimizer=None, synchronize: bool = True) -> dict:
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
    return state.get("extra", {})
