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
    host_names: tuple = ()        # host name of every world rank (gathered once at start)
    push_seq: dict = {}           # parent members -> number of splits made from that communicator


S = State()
plan_cache: dict = {}       # derived from communicators / span / tunables; cleared when any of them changes


def _require_started() -> None:
    if not S.started:
        raise RuntimeError("torchmpi_b200.start() has not been called")
    from . import watchdog
    watchdog.check()          # a lost peer or an expired wait poisons the job: fail at once, do not wait again


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


def _ensure_groups(member_lists, world_collective: bool) -> None:
    """Makes the groups of a new communicator level.

    ``world_collective``: the split was made by every rank of the job at once (the parent is the world), so
    ordinary process groups can be created, by all ranks in one global order, for ALL groups of the split.
    Otherwise only the members are here: the groups of this rank become ``gdist.LightGroup`` objects."""
    from .gdist import LightGroup
    if world_collective:
        for m in sorted({tuple(m) for m in member_lists if 1 < len(m) < S.world}):
            if m not in S.groups or isinstance(S.groups[m], LightGroup):
                S.groups[m] = dist.new_group(list(m), backend=_backend_string())
        return
    for m in member_lists:
        m = tuple(m)
        if 1 < len(m) < S.world and S.rank in m and m not in S.groups:
            S.groups[m] = LightGroup(m, S.rank)


def _all_groups_of_split(parent, keys, cartesian_wanted: bool):
    """Every intra and inter group of the split of ``parent`` by ``keys`` (one key per parent member), the way
    ``tmpi_comm_push`` forms them: groups in sorted-key order, members in parent order."""
    order = sorted(range(len(parent)), key=lambda i: (keys[i], i))
    groups, last = [], None
    for i in order:
        if keys[i] != last:
            groups.append([])
            last = keys[i]
        groups[-1].append(parent[i])
    same = all(len(g) == len(groups[0]) for g in groups)
    out = [tuple(g) for g in groups]
    if same and cartesian_wanted:
        out += [tuple(g[j] for g in groups) for j in range(len(groups[0]))]
    else:
        out.append(tuple(g[0] for g in groups))
    # inter groups list their members in parent order
    pos = {r: i for i, r in enumerate(parent)}
    return [tuple(sorted(g, key=lambda r: pos[r])) for g in out]


def _store():
    from torch.distributed import distributed_c10d
    return distributed_c10d._get_default_store()


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


def group_of(level: int, world_rank: int) -> tuple:
    """Members (world ranks, group order) of the group that ``world_rank`` joined in the split at ``level``; ``()``
    when that rank was not part of the split."""
    buf = (C.c_int * MAX_WORLD)()
    n = lib.tmpi_comm_group_of(int(level), int(world_rank), buf, MAX_WORLD)
    if n < 0:
        check(-n)
    return tuple(buf[i] for i in range(n))


def intra_members(level: int) -> tuple:
    return _members(level, False)


def inter_members(level: int) -> tuple:
    return _members(level, True)


def push_communicator(key: str) -> int:
    """Splits the communicator under the cursor by ``key`` and descends into the new level.

    Ranks with equal keys form the new intra group.  Only the members of the current communicator make
    this call (each with its own key), as in the reference (lib/c_api.h:42-47,
    lib/resources.cpp:187-350): the keys travel through the job's key-value store under a name scoped by
    the parent communicator, and the process groups of the new level are created by their members alone.
    Returns the new level.
    """
    _require_started()
    key = str(key)
    if len(key.encode()) >= KEY_LEN:
        raise ValueError(f"communicator key longer than {KEY_LEN - 1} bytes")
    parent = current_members()
    keys = bytearray(KEY_LEN * len(parent))
    all_keys = [key]
    if len(parent) > 1:
        seq = S.push_seq.get(parent, 0)
        S.push_seq[parent] = seq + 1
        prefix = f"tmpi/{S.job_id}/push/{'.'.join(map(str, parent))}/{seq}/"
        store = _store()
        store.set(prefix + str(S.rank), key)
        for i, r in enumerate(parent):
            kb = key.encode() if r == S.rank else bytes(store.get(prefix + str(r)))      # blocks until rank r has pushed
            keys[i * KEY_LEN:i * KEY_LEN + len(kb)] = kb
        all_keys = [bytes(keys[i * KEY_LEN:(i + 1) * KEY_LEN]).rstrip(b"\0").decode() for i in range(len(parent))]
    else:
        kb = key.encode()
        keys[:len(kb)] = kb
    level = lib.tmpi_comm_push(bytes(keys), _lib.int_array(parent), len(parent), key.encode())
    if level < 0:
        check(level)
    if len(parent) == S.world:
        from . import config
        cart = bool(config.get("use_cartesian_communicator"))
        _ensure_groups(_all_groups_of_split(parent, all_keys, cart), world_collective=True)
    else:
        _ensure_groups([intra_members(level), inter_members(level)], world_collective=False)
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
    return len({S.host_names[r] for r in current_members()})      # host names were gathered once at start


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
        from . import gdist
        gdist.all_reduce(torch.zeros(1), g)
