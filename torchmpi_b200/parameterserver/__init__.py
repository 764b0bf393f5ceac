"""Sharded parameter server (reference: lib/parameterserver.cpp, torchmpi/parameterserver/init.lua).

``init(t)`` shards a tensor over the ranks of the communicator under the cursor:
``floor(n / size)`` elements each, the first ``n mod size`` ranks one more,
contiguous and rank ordered.  ``send(ps, t, rule)`` applies ``rule`` (``'zero'``,
``'copy'`` or ``'add'``) with this rank's ``t`` to every shard; ``receive(ps, t)``
gathers all shards into ``t``.  Both are asynchronous and return a handle.

Where the reference keeps shards in host memory and serves MPI messages from a
polling thread, shards here live in a symmetric heap - GPU memory for CUDA
tensors, shared memory for CPU tensors - and a client updates or reads them
*one-sidedly*: a kernel (or a pool thread on the CPU) stores, adds or loads
directly in the owner's memory.  When the handle of a ``send`` has completed the
update is already in place at every owner, so ``sync_handle(send); barrier()``
still means "visible to everybody" (lib/parameterserver.cpp:339-341).
Concurrent ``add`` updates are exact (atomic adds on the GPU, a per-shard lock on
the CPU); a ``copy``/``zero`` racing with other updates on the GPU is resolved
per element, so separate them with a barrier as the reference's tests do - or pass
``serialized=True`` to ``send``: such sends to one server are applied one whole
message at a time across all clients (a ticket lock in the rendezvous store; the
call returns when the update is in place), which is the reference's guarantee that
a shard never sees two rules interleaved (lib/parameterserver.cpp:426-499, one
message at a time per shard) at the price of a blocking call.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from .. import _lib, cache, config, runtime
from .._lib import lib, check, dtype_code
from ..handles import Handle, sync_handle, sync_handles as _sync_handles
from ..runtime import S

RULES = {"zero": 0, "copy": 1, "add": 2}
_live: List["ParameterServer"] = []
_created = {}          # members -> servers created so far over exactly these members (the same on each of them)


def shard_range(n: int, size: int, rank: int):
    """[begin, end) of rank's shard of n elements."""
    q, r = divmod(n, size)
    b = rank * q + min(rank, r)
    return b, b + q + (1 if rank < r else 0)


class ParameterServer:
    """One sharded tensor.  Created collectively by ``init``."""

    def __init__(self, t: torch.Tensor):
        runtime._require_started()
        if not t.is_contiguous():
            raise ValueError("parameter server tensors must be contiguous")
        self.members = runtime.current_members()
        self.me = self.members.index(S.rank)
        self.n = t.numel()
        self.dtype = t.dtype
        if self.n < len(self.members):
            raise ValueError("parameter server needs at least one element per rank")
        self.on_gpu = bool(t.is_cuda and S.cuda_heap is not None and S.cuda_heap.covers(self.members))
        self.freed = False
        # a name every member derives alike: creation is collective over the members, in the same order on each
        key = tuple(self.members)
        serial = _created[key] = _created.get(key, 0) + 1
        self.uid = f"{min(key)}.{len(key)}.{hash(key) & 0xffffffff:x}.{serial}"
        self._arr = _lib.int_array(self.members)
        self._staging = None
        runtime.barrier()
        if self.on_gpu:
            self.impl = S.cuda_heap.ps_create(t, self.members)
        else:
            if not (S.shm_ready and all(m in S.shm_ranks for m in self.members)):
                raise RuntimeError("parameter server: the ranks of this communicator share no heap "
                                   "(host shared memory is unavailable)")
            host = t.detach().cpu() if t.is_cuda else t
            r = lib.tmpi_shm_ps_init(host.data_ptr(), self.n, dtype_code(t.dtype), self._arr, len(self.members), self.me)
            if r < 0:
                check(r)
            self.impl = r
        runtime.barrier()
        _live.append(self)

    # ---- client operations
    def send(self, t: torch.Tensor, rule: str = "add", serialized: bool = False) -> Handle:
        if rule not in RULES:
            raise ValueError(f"unknown update rule '{rule}' (expected one of {sorted(RULES)})")
        self._check(t)
        if serialized:
            return self._send_serialized(t, rule)
        if config.get("fault_drop_ps_requests"):      # host-side fault injection: the request never reports back
            return Handle(ids=[lib.tmpi_test_lost_handle()])
        if self.on_gpu:
            return S.cuda_heap.ps_push(self.impl, t, RULES[rule])
        host = self._to_host(t)
        return Handle(ids=[lib.tmpi_shm_ps_send(self.impl, host.data_ptr(), RULES[rule])], keep=(host,))

    def _send_serialized(self, t: torch.Tensor, rule: str) -> Handle:
        """One whole message at a time across all clients of this server: take a ticket, wait for the turn, apply the
        update, wait until it is in place at every owner, pass the turn on.  Returns a completed handle."""
        import time
        from .. import watchdog
        store = runtime._store()
        base = f"tmpi/ps/{self.uid}"
        ticket = store.add(base + "/ticket", 1)
        budget_s = config.get("handle_wait_budget_ms") / 1e3
        t0, pause = time.monotonic(), 1e-4
        while store.add(base + "/serving", 0) != ticket - 1:
            watchdog.check()
            if time.monotonic() - t0 > budget_s:
                watchdog.poison(f"parameter server {self.uid}: the turn of ticket {ticket} never came")
                raise _lib.TimeoutError_(_lib.ERR_TIMEOUT, "serialized parameter-server send timed out waiting for its turn")
            time.sleep(pause)
            pause = min(pause * 2, 2e-3)
        try:
            self.send(t, rule).wait()
        finally:
            store.add(base + "/serving", 1)
        return Handle()

    def receive(self, t: torch.Tensor) -> Handle:
        self._check(t)
        if config.get("fault_drop_ps_requests"):
            return Handle(ids=[lib.tmpi_test_lost_handle()])
        if self.on_gpu:
            return S.cuda_heap.ps_pull(self.impl, t)
        if t.is_cuda:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            return Handle(ids=[lib.tmpi_shm_ps_receive(self.impl, host.data_ptr())],
                          finalizers=[lambda: t.copy_(host, non_blocking=False)], keep=(host,))
        return Handle(ids=[lib.tmpi_shm_ps_receive(self.impl, t.data_ptr())], keep=(t,))

    def free(self, collective: bool = True) -> None:
        if self.freed:
            return
        if collective:
            runtime.barrier()
        if self.on_gpu:
            S.cuda_heap.ps_free(self.impl)
        else:
            lib.tmpi_shm_ps_free(self.impl)
        self.freed = True
        if self in _live:
            _live.remove(self)
        if collective:
            runtime.barrier()

    def _check(self, t):
        if self.freed:
            raise RuntimeError("parameter server already freed")
        if t.numel() != self.n or t.dtype != self.dtype or not t.is_contiguous():
            raise ValueError("tensor does not match the parameter server (numel, dtype, contiguity)")

    def _to_host(self, t):
        if not t.is_cuda:
            return t
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        host.copy_(t, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return host


def init(t: torch.Tensor) -> ParameterServer:
    return ParameterServer(t)


def send(ps: ParameterServer, t: torch.Tensor, rule: str = "add", serialized: bool = False) -> Handle:
    return ps.send(t, rule, serialized)


def receive(ps: ParameterServer, t: torch.Tensor) -> Handle:
    return ps.receive(t)


def free(ps: ParameterServer) -> None:
    ps.free()


def free_all(collective: bool = True) -> None:
    for ps in list(_live):
        ps.free(collective=collective)
    cache.parameter_servers.clear()


def sync_handles(hs: Sequence[Optional[Handle]]) -> list:
    _sync_handles(hs)
    return []


# ---------------------------------------------------------------- helpers on lists of tensors
def init_tensors(tensors: Sequence[torch.Tensor], prefetch_allocator: Optional[Callable] = None,
                 ps_init_fun: Optional[Callable] = None) -> None:
    """Creates one server per tensor with a prefetch clone; rank 0 seeds it with ``copy``."""
    for t in tensors:
        if cache.key(t) in cache.parameter_servers:
            continue
        # the prefetch clone starts as a copy of the tensor: the first integration may come before
        # the first prefetch (update.lua: integrate at delay + f, prefetch at delay + f + prefetch)
        pre = prefetch_allocator(t) if prefetch_allocator else t.detach().clone()
        cache.prefetch_tensor_references[cache.key(t)] = pre
        ps = init(t)
        cache.parameter_servers[cache.key(t)] = (t, ps)
        if ps_init_fun is not None:
            ps_init_fun(ps, t)
        elif runtime.rank() == 0:
            sync_handle(send(ps, t, "copy"))
        runtime.barrier()


def prefetch_tensors(tensors: Sequence[torch.Tensor]) -> List[Handle]:
    """Starts fetching every tensor's current server value into its prefetch clone."""
    return [receive(cache.parameter_servers[cache.key(t)][1], cache.prefetch_tensor_references[cache.key(t)]) for t in tensors]


def integrate_tensors(tensors: Sequence[torch.Tensor], fn: Callable[[torch.Tensor, torch.Tensor], None]) -> None:
    """Calls ``fn(prefetched, t)`` for every tensor."""
    with torch.no_grad():
        for t in tensors:
            fn(cache.prefetch_tensor_references[cache.key(t)], t)


def send_tensors(tensors: Sequence[torch.Tensor], updates: Sequence[torch.Tensor], rule: str = "add",
                 preprocess: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> List[Handle]:
    """Sends ``updates[i]`` to the server of ``tensors[i]``; ``preprocess`` (e.g. scaling by -lr) is
    applied to a staging copy, never to the caller's tensor."""
    hs = []
    with torch.no_grad():
        for t, u in zip(tensors, updates):
            if preprocess is not None:
                st = cache.send_tensor_references.get(cache.key(t))
                if st is None or st.shape != u.shape:
                    st = cache.send_tensor_references[cache.key(t)] = torch.empty_like(u)
                st.copy_(u)
                u = preprocess(st)
                u = st if u is None else u
            hs.append(send(cache.parameter_servers[cache.key(t)][1], u, rule))
    return hs


from .update import Update  # noqa: E402
from .downpour import DownpourUpdate  # noqa: E402
from .easgd import EASGDUpdate  # noqa: E402

initTensors, prefetchTensors, integrateTensors, sendTensors, syncHandles, syncHandle, freeAll = (
    init_tensors, prefetch_tensors, integrate_tensors, send_tensors, sync_handles, sync_handle, free_all)
