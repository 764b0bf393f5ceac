"""torchmpi_b200: a Blackwell-native distributed-training runtime with TorchMPI's capabilities.

Public surface (reference: torchmpi/init.lua): ``start / stop / rank / size /
barrier / communicator_names``; tensor collectives ``broadcast_tensor,
reduce_tensor, allreduce_tensor, sendreceive_tensor, allgather_tensor`` in the
namespaces ``mpi`` (selector-chosen backend), ``mpi.async_``, ``mpi.p2p``,
``mpi.async_.p2p``, ``mpi.nccl``, ``mpi.async_.nccl``, ``mpi.gloo``,
``mpi.async_.gloo``; scalar collectives ``allreduce_double`` ...; ``sync_handle``;
``check_with_allreduce``; the selector; ``nn``, ``engine``, ``BlockSequential``,
``parameterserver`` and the ``Update`` policies.  Every snake_case name has the
reference's camelCase alias (``allreduceTensor`` ...).
"""
from __future__ import annotations

import types as _types

import torch as _torch

from . import _lib, config
from ._lib import TorchMPIError, TimeoutError_ as TimeoutError  # noqa: A001
from .watchdog import CommunicatorPoisoned
from .bootstrap import start, stop
from .runtime import (S as _S, barrier, rank, size, world_rank, world_size, communicator_names,
                      push_communicator, set_communicator, set_collective_span, collective_span,
                      is_cartesian_communicator, num_nodes_in_communicator, set_cartesian_communicator,
                      set_tree_communicator, communicator_level, current_members, intra_members,
                      inter_members)
from .collectives import (allreduce_tensor, broadcast_tensor, reduce_tensor, sendreceive_tensor,
                          allgather_tensor, reduce_scatter_tensor)
from .handles import Handle, sync_handle, sync_handles, sync_all
from .selector import collective_selector_to_string, collective_availability
from . import selector as _selector
from .scalars import *  # noqa: F401,F403 - allreduce_double, broadcast_int, ...
from .scalars import check_with_allreduce
from . import scalars as _scalars


def _ns(backend, async_op, ops):
    """A namespace of tensor collectives bound to one backend and sync/async flavour."""
    ns = _types.SimpleNamespace()
    table = {
        "allreduce_tensor": lambda inp, out=None, **kw: allreduce_tensor(inp, out, backend=backend, async_op=async_op, **kw),
        "broadcast_tensor": lambda root, t, **kw: broadcast_tensor(root, t, backend=backend, async_op=async_op, **kw),
        "reduce_tensor": lambda root, inp, out=None, **kw: reduce_tensor(root, inp, out, backend=backend, async_op=async_op, **kw),
        "sendreceive_tensor": lambda t, src, dst, **kw: sendreceive_tensor(t, src, dst, backend=backend, **kw),
        "allgather_tensor": lambda inp, out, **kw: allgather_tensor(inp, out, backend=backend, **kw),
    }
    for name in ops:
        fn = table[name]
        setattr(ns, name, fn)
        head, _ = name.split("_")
        setattr(ns, head + "Tensor", fn)
    return ns


_ALL = ["allreduce_tensor", "broadcast_tensor", "reduce_tensor", "sendreceive_tensor", "allgather_tensor"]
p2p = _ns("p2p", False, ["allreduce_tensor", "broadcast_tensor", "reduce_tensor", "allgather_tensor"])
nccl = _ns("nccl", False, ["allreduce_tensor", "broadcast_tensor", "reduce_tensor"])
gloo = _ns("gloo", False, ["allreduce_tensor", "broadcast_tensor"])
async_ = _ns(None, True, ["allreduce_tensor", "broadcast_tensor", "reduce_tensor"])
async_.p2p = _ns("p2p", True, ["allreduce_tensor", "broadcast_tensor", "reduce_tensor"])
async_.nccl = _ns("nccl", True, ["allreduce_tensor", "broadcast_tensor", "reduce_tensor"])
async_.gloo = _ns("gloo", True, ["allreduce_tensor", "broadcast_tensor"])
async_.streams = None


def _init_streams(use_async: bool = True):
    """Reserves the side streams of the async paths (``mpi.async.initStreams``, torchmpi/init.lua:17-27)."""
    if not _S.with_cuda:
        async_.streams = _types.SimpleNamespace(default=None, copy_to_gpu=None, copy_to_cpu=None,
                                                local_collective=None, global_collective=None)
        return async_.streams
    mk = (lambda: _torch.cuda.Stream(priority=-1)) if use_async else (lambda: _torch.cuda.current_stream())
    async_.streams = _types.SimpleNamespace(default=_torch.cuda.current_stream(), copy_to_gpu=mk(),
                                            copy_to_cpu=mk(), local_collective=mk(), global_collective=mk())
    return async_.streams


async_.init_streams = async_.initStreams = _init_streams

# camelCase aliases of the reference
allreduceTensor, broadcastTensor, reduceTensor = allreduce_tensor, broadcast_tensor, reduce_tensor
sendreceiveTensor, allgatherTensor = sendreceive_tensor, allgather_tensor
syncHandle, communicatorNames, checkWithAllreduce = sync_handle, communicator_names, check_with_allreduce
collectiveSelectorToString, collectiveAvailability = collective_selector_to_string, collective_availability

# raw communicator calls under their C names (lib/c_api.h:37-66)
C = _types.SimpleNamespace(
    torchmpi_push_communicator=push_communicator,
    torchmpi_set_communicator=set_communicator,
    torchmpi_set_collective_span=set_collective_span,
    torchmpi_is_cartesian_communicator=is_cartesian_communicator,
    torchmpi_num_nodes_in_communicator=num_nodes_in_communicator,
    torchmpi_set_tree_communicator=set_tree_communicator,
    torchmpi_set_cartesian_communicator=set_cartesian_communicator,
    torchmpi_free_ipc_descriptors=lambda: None,   # peers are mapped once per heap; nothing per tensor to free
    torchmpi_set_flat_collectives=config.set_flat_collectives,
    torchmpi_set_hierarchical_collectives=config.set_hierarchical_collectives,
    torchmpi_set_staged_collectives=config.set_staged_collectives,
    torchmpi_set_direct_collectives=config.set_direct_collectives,
)

_CONSTANTS = {
    "with_cuda": lambda: _S.with_cuda, "withCuda": lambda: _S.with_cuda,
    "has_nccl": lambda: _S.with_cuda, "hasNCCL": lambda: _S.with_cuda,
    "has_gloo": lambda: True, "hasGloo": lambda: True,
    "has_gloo_cuda": lambda: _S.with_cuda, "hasGlooCuda": lambda: _S.with_cuda,
    "ipc_groups": lambda: _S.ipc_groups, "ipcGroups": lambda: _S.ipc_groups,
    "single_ipc_group": lambda: _S.single_ipc_group, "singleIPCGroup": lambda: _S.single_ipc_group,
    "host_name": lambda: _S.host_name, "hostName": lambda: _S.host_name,
    "device": lambda: _S.device,
    "num_communicators": lambda: _S.num_communicators, "numCommunicators": lambda: _S.num_communicators,
    "need_inter_node_collectives": lambda: _S.need_inter_node_collectives,
    "needInterNodeCollectives": lambda: _S.need_inter_node_collectives,
    "collective_selector": lambda: _selector.collective_selector,
    "collectiveSelector": lambda: _selector.collective_selector,
    "started": lambda: _S.started,
}

_LAZY = {"nn", "engine", "parameterserver", "cache", "tester", "launch", "models", "ops", "parallel", "utils"}


def __getattr__(name):
    if name in _CONSTANTS:
        return _CONSTANTS[name]()
    if name in _LAZY:
        import importlib
        return importlib.import_module(f".{name}", __name__)
    if name in ("BlockSequential",):
        from .parallel.block_sequential import BlockSequential
        return BlockSequential
    if name in ("AllReduceSGDEngine",):
        from .engine import AllReduceSGDEngine
        return AllReduceSGDEngine
    if name in ("Update", "DownpourUpdate", "EASGDUpdate"):
        from . import parameterserver as _ps
        return getattr(_ps, name)
    raise AttributeError(f"module 'torchmpi_b200' has no attribute '{name}'")
