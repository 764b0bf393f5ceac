"""``start`` / ``stop``: bring the process into the job and take it out again.

Follows the sequence of the reference's ``mpi.start`` (torchmpi/init.lua:31-100):
record the host name, choose tree or cartesian communicators, create level 0,
pin the GPU by local rank, run the user's communicator hook, push the per-node
level, set the collective span and configure the selector - with a
``torch.distributed`` store/gloo control plane in place of MPI, and symmetric
heaps (host shared memory, CUDA peer memory) in place of per-tensor IPC handles.
"""
from __future__ import annotations

import ctypes as C
import datetime
import logging
import os
import socket
import uuid
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib, runtime
from ._lib import lib, check
from .runtime import S

log = logging.getLogger("torchmpi_b200")


def _env_int(*names, default=0) -> int:
    for n in names:
        v = os.environ.get(n)
        if v not in (None, ""):
            return int(v)
    return default


def _init_process_group(with_cuda: bool) -> None:
    if dist.is_initialized():
        S.owns_process_group = False
        return
    S.owns_process_group = True
    world = _env_int("WORLD_SIZE", default=1)
    rank = _env_int("RANK", default=0)
    timeout = datetime.timedelta(seconds=_env_int("TORCHMPI_TIMEOUT_S", default=600))
    backend = "cpu:gloo,cuda:nccl" if with_cuda else "gloo"
    if world == 1 and "MASTER_ADDR" not in os.environ:
        dist.init_process_group(backend, store=dist.HashStore(), rank=0, world_size=1, timeout=timeout)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend, rank=rank, world_size=world, timeout=timeout)


def _setup_host_heap() -> None:
    """Creates this rank's shared-memory segment and maps the peers on the same host."""
    names = [None] * S.world
    seg = f"/tmpi_{S.job_id}_{S.rank}"
    nbytes = _env_int("TORCHMPI_HOST_HEAP_BYTES", default=64 << 20)
    try:
        check(lib.tmpi_shm_create(seg.encode(), nbytes, S.rank, S.world, None))
        mine = (S.host_name, seg)
    except _lib.TorchMPIError as e:  # e.g. /dev/shm unavailable: stay on gloo
        log.warning("host heap unavailable: %s", e)
        mine = (S.host_name, None)
    dist.all_gather_object(names, mine)
    ok = mine[1] is not None
    peers = [r for r, (h, n) in enumerate(names) if h == S.host_name and n is not None]
    if ok:
        for r in peers:
            if r != S.rank:
                try:
                    check(lib.tmpi_shm_attach(r, names[r][1].encode()))
                except _lib.TorchMPIError as e:
                    log.warning("cannot map host heap of rank %d: %s", r, e)
                    ok = False
    flags = [None] * S.world
    dist.all_gather_object(flags, ok)
    S.shm_ranks = tuple(r for r in peers if flags[r])
    S.shm_ready = ok and len(S.shm_ranks) == len(peers)


def start(with_cuda: Optional[bool] = None,
          with_ipc_groups: bool = True,
          custom_communicator_init: Optional[Callable[[], int]] = None,
          with_cartesian_communicator: bool = False,
          collective_communicator: Optional[Callable[[], None]] = None) -> None:
    """Joins the job.  Reads ``RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT``.

    ``custom_communicator_init`` may push user communicator levels (and returns
    the level to descend into); ``collective_communicator`` runs after the
    per-node level exists and may set the collective span - the reference tests
    an undefined variable there and never calls it (torchmpi/init.lua:93-97).
    """
    if S.started:
        raise RuntimeError("torchmpi_b200.start() called twice")
    if with_cuda is None:
        with_cuda = torch.cuda.is_available()
    if with_cuda and not torch.cuda.is_available():
        raise RuntimeError("start(with_cuda=True) but no CUDA device is visible")
    S.with_cuda = bool(with_cuda)
    S.host_name = socket.gethostname()
    S.local_rank = _env_int("LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "MV2_COMM_WORLD_LOCAL_RANK", default=0)
    if S.with_cuda:
        dev = S.local_rank % torch.cuda.device_count()
        torch.cuda.set_device(dev)
        S.device = torch.device("cuda", dev)
    else:
        S.device = torch.device("cpu")
    _init_process_group(S.with_cuda)
    S.rank, S.world = dist.get_rank(), dist.get_world_size()
    if S.world > runtime.MAX_WORLD:
        raise RuntimeError(f"world size {S.world} exceeds the supported maximum {runtime.MAX_WORLD}")
    S.groups = {}
    check(lib.tmpi_set_tunable(b"use_cartesian_communicator", 1 if with_cartesian_communicator else 0))
    check(lib.tmpi_comm_reset(S.rank, S.world))
    runtime.plan_cache.clear()
    S.started = True

    jid = [uuid.uuid4().hex[:12] if S.rank == 0 else None]
    dist.broadcast_object_list(jid, src=0)
    S.job_id = jid[0]
    names = [None] * S.world
    dist.all_gather_object(names, S.host_name)
    S.host_names = tuple(names)
    S.push_seq = {}
    _setup_host_heap()

    if S.with_cuda:
        from .parallel import symm_heap
        S.cuda_heap = symm_heap.create_default_heap()

    if custom_communicator_init is not None:
        level = custom_communicator_init()
        if level is not None:
            runtime.set_communicator(int(level))

    # per-node level: ranks of one host that can reach each other's memory
    entry = runtime.communicator_level()
    S.ipc_groups = bool(with_ipc_groups)
    key = S.host_name
    if S.with_cuda and with_ipc_groups:
        from .parallel import symm_heap
        reach, S.single_ipc_group = symm_heap.peer_access_string()
        key = f"{S.host_name} cuda p2p group({reach})"
    level = runtime.push_communicator(key)
    runtime.set_collective_span(entry, level)
    runtime.set_communicator(entry)
    S.need_inter_node_collectives = runtime.num_nodes_in_communicator() > 1
    if collective_communicator is not None:
        collective_communicator()
    from . import selector, watchdog
    selector.configure()
    runtime.barrier()
    watchdog.reset()
    watchdog.start()
    if S.rank == 0:
        log.info("communicators:\n%s", runtime.communicator_names())


def stop() -> None:
    """Drains asynchronous work, frees parameter servers and heaps, leaves the job."""
    if not S.started:
        return
    from . import watchdog
    lost = watchdog.poisoned()
    watchdog.stop(goodbye=True)
    watchdog.reset()              # the teardown below must run even after a failure
    try:
        check(lib.tmpi_comm_set_typed(0, 0))
        if S.with_cuda:
            torch.cuda.synchronize()
        if lost is None:
            runtime.barrier()
    except Exception as e:  # a dead peer must not stop our own cleanup
        log.warning("stop(): barrier failed: %s", e)
    lib.tmpi_sync_all()
    from . import parameterserver, cache
    parameterserver.free_all(collective=False)
    cache.free_all_tensor_references()
    if S.cuda_heap is not None:
        try:
            if lost is None:
                runtime.barrier()
        except Exception:
            pass
        S.cuda_heap.destroy()
        S.cuda_heap = None
    lib.tmpi_shm_ps_free_all()
    lib.tmpi_shm_destroy()
    S.shm_ready = False
    if S.owns_process_group and not os.environ.get("FB_INFRA"):
        dist.destroy_process_group()
    S.groups = {}
    S.started = False
