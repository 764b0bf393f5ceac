"""Process bootstrap, teardown and the communicator stack.

One Python process drives one GPU (or is a CPU rank).  The control plane is
``torch.distributed`` (store + gloo); the data plane is the symmetric heaps of
the native runtime.  This module is the counterpart of ``mpi.start/stop`` and of
the raw communicator calls of the reference (torchmpi/init.lua:31-122,417-461;
lib/torch_mpi.cpp:231-352), without MPI.
"""
from __future__ import annotations

import ctypes as C
import datetime
import logging
import os
import socket
import uuid
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib
from ._lib import lib, check

log = logging.getLogger("torchmpi_b200")

KEY_LEN = 1024
MAX_WORLD = 64


class State:
    started = False
    rank = 0
    world = 1
    local_rank = 0
    with_cuda = False
    device: Optional[torch.device] = None
    host_name = ""
    owns_process_group = False
    groups: dict = {}             # tuple(world ranks) -> ProcessGroup
    shm_ready = False
    shm_ranks: tuple = ()         # world ranks attached to the host heap
    cuda_heap = None              # parallel.symm_heap.CudaHeap
    single_ipc_group = True
    ipc_groups = False
    need_inter_node_collectives = False
    num_communicators = 1
    job_id = ""


S = State()
plan_cache: dict = {}       # derived from communicators / span / tunables; cleared when any of them changes


def _require_started() -> None:
    if not S.started:
        raise RuntimeError("torchmpi_b200.start() has not been called")


# ---------------------------------------------------------------- groups
def group_for(members: Sequence[int]):
    """ProcessGroup of exactly these world ranks (None for a singleton)."""
    members = tuple(members)
    if len(members) <= 1:
        return None
    if len(members) == S.world:
        return dist.group.WORLD
    try:
        return S.groups[members]
    except KeyError:
        raise RuntimeError(f"no process group for ranks {members}; communicators are created with push_communicator") from None


def _ensure_groups(all_member_lists) -> None:
    """Collective over the world: creates the missing groups in one global order."""
    wanted = sorted({tuple(m) for m in all_member_lists if 1 < len(m) < S.world})
    for m in wanted:
        if m not in S.groups:
            S.groups[m] = dist.new_group(list(m), backend=_backend_string())


def _backend_string() -> str:
    return "cpu:gloo,cuda:nccl" if S.with_cuda else "gloo"


# ---------------------------------------------------------------- communicator stack
def _members(level: int, inter: bool) -> tuple:
    buf = (C.c_int * MAX_WORLD)()
    n = lib.tmpi_comm_members(level, 1 if inter else 0, buf, MAX_WORLD)
    if n < 0:
        check(n)
    return tuple(buf[i] for i in range(n))


def current_members() -> tuple:
    """World ranks of the communicator under the cursor, in communicator-rank order."""
    _require_started()
    buf = (C.c_int * MAX_WORLD)()
    n = lib.tmpi_comm_current_members(buf, MAX_WORLD)
    if n < 0:
        check(n)
    return tuple(buf[i] for i in range(n))


def intra_members(level: int) -> tuple:
    return _members(level, False)


def inter_members(level: int) -> tuple:
    return _members(level, True)


def push_communicator(key: str) -> int:
    """Splits the communicator under the cursor by ``key`` and descends into the new level.

    Ranks with equal keys form the new intra group.  Every rank of the world has
    to make this call at the same point of the program (with its own key), since
    process groups are created collectively; the reference only requires the
    members of the current communicator (lib/c_api.h:42-47).
    Returns the new level.
    """
    _require_started()
    key = str(key)
    if len(key.encode()) >= KEY_LEN:
        raise ValueError(f"communicator key longer than {KEY_LEN - 1} bytes")
    parent = current_members()
    table = [None] * S.world
    dist.all_gather_object(table, (parent, key))
    keys = bytearray(KEY_LEN * len(parent))
    for i, r in enumerate(parent):
        p, k = table[r]
        if tuple(p) != parent:
            raise RuntimeError(f"rank {r} pushed a communicator from a different parent {p} than rank {S.rank} ({parent})")
        kb = k.encode()
        keys[i * KEY_LEN:i * KEY_LEN + len(kb)] = kb
    level = lib.tmpi_comm_push(bytes(keys), _lib.int_array(parent), len(parent), key.encode())
    if level < 0:
        check(level)
    mine = (intra_members(level), inter_members(level))
    everyone = [None] * S.world
    dist.all_gather_object(everyone, mine)
    _ensure_groups([g for pair in everyone for g in pair])
    S.num_communicators = lib.tmpi_comm_num_levels()
    plan_cache.clear()
    return level


def set_communicator(level: int, inter: bool = False) -> None:
    _require_started()
    check(lib.tmpi_comm_set_typed(int(level), 1 if inter else 0))


def communicator_level() -> int:
    return lib.tmpi_comm_level()


def set_collective_span(begin: int, end: int) -> None:
    _require_started()
    check(lib.tmpi_comm_set_span(int(begin), int(end)))
    plan_cache.clear()


def collective_span() -> tuple:
    b, e = C.c_int(), C.c_int()
    lib.tmpi_comm_get_span(C.byref(b), C.byref(e))
    return b.value, e.value


def is_cartesian_communicator(level: int = -1) -> bool:
    _require_started()
    r = lib.tmpi_comm_is_cartesian(level)
    if r < 0:
        check(r)
    return bool(r)


def set_cartesian_communicator() -> None:
    check(lib.tmpi_set_tunable(b"use_cartesian_communicator", 1))
    plan_cache.clear()


def set_tree_communicator() -> None:
    check(lib.tmpi_set_tunable(b"use_cartesian_communicator", 0))
    plan_cache.clear()


def communicator_names() -> str:
    _require_started()
    buf = C.create_string_buffer(1 << 16)
    lib.tmpi_comm_names(buf, len(buf))
    return buf.value.decode()


def num_nodes_in_communicator() -> int:
    """Number of distinct hosts among the ranks of the current communicator.

    Hosts are counted as a set; the reference de-duplicates without sorting and is
    only right when ranks are grouped by host (lib/torch_mpi.cpp:338-342).
    """
    _require_started()
    members = current_members()
    names = [None] * S.world
    dist.all_gather_object(names, S.host_name)
    return len({names[r] for r in members})


def rank() -> int:
    """Rank inside the communicator under the cursor."""
    _require_started()
    return current_members().index(S.rank)


def size() -> int:
    _require_started()
    return len(current_members())


def world_rank() -> int:
    return S.rank


def world_size() -> int:
    return S.world


def barrier() -> None:
    """Barrier over the communicator under the cursor."""
    _require_started()
    g = group_for(current_members())
    if g is not None:
        # a host barrier on the gloo side of the group (the control plane), like MPI_Barrier
        dist.all_reduce(torch.zeros(1), group=g)
