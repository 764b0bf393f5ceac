"""Python side of the CUDA symmetric heap.

``CudaHeap`` creates this rank's slab, exchanges the mapping blobs over the
control plane, binds the NVLink multicast object when the device has one, hands
out symmetric allocations as torch tensors, and wraps the collective entry
points of the native runtime.  It stands where the reference keeps per-tensor
IPC descriptors and event matrices (lib/resources.cpp:840-1163).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import _lib, config
from .._lib import lib, check, dtype_code, stream_ptr, Group, SgdBucket
from ..handles import Handle

LANE_SYNC, LANE_ASYNC, LANE_OPT, LANE_PS = 0, 1, 2, 3


class _RawCudaBuffer:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def peer_access_string():
    """("0-1-2-...", single_group): the devices this rank's GPU can peer-access, itself included."""
    me = torch.cuda.current_device()
    n = torch.cuda.device_count()
    reach = [d for d in range(n) if d == me or torch.cuda.can_device_access_peer(me, d)]
    return "-".join(str(d) for d in reach), len(reach) == n


class CudaHeap:
    def __init__(self, world_rank: int, world: int, heap_bytes: int, backend: int, emulated: bool = False):
        self.rank, self.world, self.emulated = world_rank, world, emulated
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.has_multicast = False
        self._ps = {}
        self._ps_next = 0
        self._keep = []
        self._layout = None
        if emulated:
            check(lib.tmpi_cuda_heap_create_emulated(heap_bytes, world))
        else:
            check(lib.tmpi_cuda_heap_create(heap_bytes, world_rank, world, backend))
        self.backend = backend

    # ---- rendezvous (collective over the world)
    def rendezvous(self) -> None:
        buf = C.create_string_buffer(256)
        n = lib.tmpi_cuda_heap_export(buf, 256)
        if n < 0:
            check(n)
        blobs = [None] * self.world
        dist.all_gather_object(blobs, bytes(buf.raw[:n]))
        for r, b in enumerate(blobs):
            if r != self.rank:
                check(lib.tmpi_cuda_heap_import(r, b, len(b)))
        check(lib.tmpi_cuda_heap_finish())
        if self.backend == 1 and self.world > 1:
            self._bind_multicast()

    def _bind_multicast(self) -> None:
        buf = C.create_string_buffer(256)
        n = lib.tmpi_cuda_heap_mc_export(buf, 256)
        blobs = [None] * self.world
        dist.all_gather_object(blobs, bytes(buf.raw[:max(0, n)]))
        blob = blobs[0]
        ok = len(blob) >= 64
        if ok:
            ok = lib.tmpi_cuda_heap_mc_import(blob, len(blob)) == 0
        flags = [None] * self.world
        dist.all_gather_object(flags, ok)            # doubles as "every device has been added"
        if all(flags):
            ok = lib.tmpi_cuda_heap_mc_bind() == 0
            dist.all_gather_object(flags, ok)
            self.has_multicast = all(flags)
            if not self.has_multicast:
                config.set("use_nvls", 0)

    def destroy(self) -> None:
        self._ps.clear()
        self._keep.clear()
        check(lib.tmpi_cuda_heap_destroy())

    # ---- allocation
    def covers(self, members: Sequence[int]) -> bool:
        return all(0 <= m < self.world for m in members)

    def base(self, peer: Optional[int] = None) -> int:
        return lib.tmpi_cuda_heap_base(self.rank if peer is None else peer) or 0

    def alloc(self, nbytes: int, align: int = 256, peer: Optional[int] = None):
        """(uint8 tensor over this rank's copy, byte offset) of a fresh symmetric allocation.
        Every rank must make the same sequence of ``alloc`` calls."""
        off = lib.tmpi_cuda_heap_alloc(nbytes, align)
        if off == C.c_size_t(-1).value:
            raise _lib.TorchMPIError(_lib.ERR_STATE, _lib.last_error())
        return self.view(off, nbytes, peer), off

    def view(self, off: int, nbytes: int, peer: Optional[int] = None) -> torch.Tensor:
        raw = _RawCudaBuffer(self.base(peer) + off, nbytes)
        t = torch.as_tensor(raw, device=self.device)
        self._keep.append(raw)
        return t

    def allocator(self):
        """``allocator(nbytes) -> (uint8 tensor, offset)`` for FlatBuckets."""
        return lambda nbytes: self.alloc(nbytes)

    def empty(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        raw, _ = self.alloc(numel * es)
        return raw.view(dtype)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base()
        if off < 0 or off + t.numel() * t.element_size() > self.layout()["total_bytes"]:
            return -1
        return off

    def layout(self) -> dict:
        """Byte offsets of the regions of one rank's mapping (one-shot slots, bounce buffers, arena)."""
        if self._layout is None:
            v = (C.c_size_t * 6)()
            check(lib.tmpi_cuda_heap_layout(v, 6))
            self._layout = dict(zip(("slots_off", "slot_bytes", "bounce_off", "bounce_bytes", "arena_off", "total_bytes"),
                                    (int(x) for x in v)))
        return self._layout

    # ---- groups
    def _group(self, members: Sequence[int], lane: int = LANE_SYNC, me: Optional[int] = None):
        arr = _lib.int_array(members)
        g = Group(arr, len(members), tuple(members).index(self.rank) if me is None else me, lane)
        return g, arr

    def check_status(self, lane: int = LANE_SYNC) -> None:
        code, where, peer = C.c_int(), C.c_int(), C.c_int()
        check(lib.tmpi_cuda_collective_status(lane, C.byref(code), C.byref(where), C.byref(peer)))
        if code.value:
            cls = _lib.TimeoutError_ if code.value == _lib.ERR_TIMEOUT else _lib.TorchMPIError
            from .. import watchdog
            watchdog.poison(f"device-side wait gave up at point {where.value} waiting for rank {peer.value}")
            raise cls(code.value, f"device-side wait gave up at point {where.value} waiting for rank {peer.value}")

    # ---- collectives on tensors
    def _needs_staging(self, t: torch.Tensor) -> bool:
        """Every rank must pick the same kernel variant (16-byte packs or single elements) without
        seeing the other ranks' pointers.  Heap offsets are symmetric, so heap tensors agree by
        construction; a tensor outside the heap agrees only if its pointer is 16-byte aligned, in
        which case the variant depends on the element count alone."""
        return t.data_ptr() % 16 != 0 and self.offset_of(t) < 0

    def allreduce(self, inp, out, members, scale=1.0, algo=0, async_op=False):
        fin, dst = [], out
        if self._needs_staging(inp) or self._needs_staging(out):
            tmp = torch.empty(inp.numel(), dtype=inp.dtype, device=inp.device).copy_(inp)
            fin, inp, out = [lambda: dst.copy_(tmp)], tmp, tmp
        g, arr = self._group(members)
        args = (inp.data_ptr(), out.data_ptr(), inp.numel(), dtype_code(inp.dtype), float(scale), C.byref(g), int(algo),
                stream_ptr())
        if async_op:
            return Handle(ids=[lib.tmpi_cuda_allreduce_async(*args)], finalizers=fin, keep=(inp, out, arr, g))
        check(lib.tmpi_cuda_allreduce(*args))
        for f in fin:
            f()
        return None

    def broadcast(self, t, root, members, async_op=False):
        fin, dst = [], t
        if self._needs_staging(t):
            tmp = torch.empty(t.numel(), dtype=t.dtype, device=t.device).copy_(t)
            fin, t = [lambda: dst.copy_(tmp)], tmp
        g, arr = self._group(members)
        args = (t.data_ptr(), t.numel(), dtype_code(t.dtype), int(root), C.byref(g), stream_ptr())
        if async_op:
            return Handle(ids=[lib.tmpi_cuda_broadcast_async(*args)], finalizers=fin, keep=(t, arr, g))
        check(lib.tmpi_cuda_broadcast(*args))
        for f in fin:
            f()
        return None

    def _staged(self, t: torch.Tensor, copy_in: bool):
        """(tensor to hand to the kernel, finalizer or None): an aligned stand-in for a tensor that
        ``_needs_staging``, so that the pack width and the grid do not depend on one rank's pointer."""
        if t.data_ptr() % 16 == 0:          # aligned on this rank: the variant then depends on counts alone
            return t, None
        tmp = torch.empty(t.numel(), dtype=t.dtype, device=t.device)
        if copy_in:
            tmp.copy_(t.reshape(-1))
        return tmp, (lambda: t.reshape(-1).copy_(tmp))

    def reduce(self, inp, out, root, members, async_op=False):
        inp, _ = self._staged(inp, True)
        out, fin = self._staged(out, False)
        g, arr = self._group(members)
        check(lib.tmpi_cuda_reduce(inp.data_ptr(), out.data_ptr(), inp.numel(), dtype_code(inp.dtype), int(root),
                                   C.byref(g), stream_ptr()))
        if fin is not None:
            fin()
        return Handle() if async_op else None

    def allgatherv(self, inp, out, counts, members):
        inp, _ = self._staged(inp, True)
        out, fin = self._staged(out, False)
        g, arr = self._group(members)
        carr = (C.c_int64 * len(counts))(*counts)
        check(lib.tmpi_cuda_allgatherv(inp.data_ptr(), out.data_ptr(), inp.numel(), carr, dtype_code(inp.dtype),
                                       C.byref(g), stream_ptr()))
        if fin is not None:
            fin()

    def reduce_scatter(self, inp, out, members, scale=1.0):
        inp, _ = self._staged(inp, True)
        out, fin = self._staged(out, False)
        g, arr = self._group(members)
        check(lib.tmpi_cuda_reduce_scatter(inp.data_ptr(), out.data_ptr(), out.numel(), dtype_code(inp.dtype),
                                           float(scale), C.byref(g), stream_ptr()))
        if fin is not None:
            fin()

    def barrier(self, members, stream=None):
        g, arr = self._group(members)
        check(lib.tmpi_cuda_barrier(C.byref(g), stream_ptr(stream)))

    # ---- fused optimizer
    def allreduce_sgd(self, bucket: SgdBucket, members, algo=0, stream=None, lane=LANE_OPT):
        g, arr = self._group(members, lane)
        check(lib.tmpi_cuda_allreduce_sgd(C.byref(bucket), C.byref(g), int(algo), stream_ptr(stream)))

    # ---- parameter server
    def ps_create(self, t: torch.Tensor, members) -> int:
        """Collective over ``members``: reserves the shard storage and seeds this rank's shard from ``t``."""
        n, N = t.numel(), len(members)
        es = t.element_size()
        cap = (n + N - 1) // N * es
        raw, off = self.alloc(cap)
        me = tuple(members).index(self.rank)
        q, r = divmod(n, N)
        b = me * q + min(me, r)
        e = b + q + (1 if me < r else 0)
        raw.view(t.dtype)[:e - b].copy_(t.detach().reshape(-1)[b:e])
        torch.cuda.current_stream().synchronize()
        pid = self._ps_next
        self._ps_next += 1
        self._ps[pid] = (off, n, t.dtype, tuple(members), raw)
        return pid

    def ps_free(self, pid: int) -> None:
        self._ps.pop(pid, None)     # the arena is a bump allocator: space returns with the heap

    def ps_push(self, pid: int, t: torch.Tensor, rule: int) -> Handle:
        off, n, dt, members, _ = self._ps[pid]
        g, arr = self._group(members, LANE_PS)
        h = lib.tmpi_cuda_ps_push_async(off, t.data_ptr(), n, dtype_code(dt), int(rule), C.byref(g), stream_ptr())
        return Handle(ids=[h], keep=(t, arr, g))

    def ps_pull(self, pid: int, t: torch.Tensor) -> Handle:
        off, n, dt, members, _ = self._ps[pid]
        g, arr = self._group(members, LANE_PS)
        h = lib.tmpi_cuda_ps_pull_async(off, t.data_ptr(), n, dtype_code(dt), C.byref(g), stream_ptr())
        return Handle(ids=[h], keep=(t, arr, g))


def create_default_heap() -> CudaHeap:
    """Heap over all ranks of the job (collective).  ``TORCHMPI_HEAP_BACKEND=ipc|vmm`` picks the
    mapping mechanism; the default tries the virtual-memory backend (needed for NVLS)."""
    from ..runtime import S
    check(lib.tmpi_cuda_set_device(S.device.index))
    backend = {"ipc": 0, "vmm": 1}[os.environ.get("TORCHMPI_HEAP_BACKEND", "vmm" if S.world > 1 else "ipc")]
    h = None
    ok = True
    try:
        h = CudaHeap(S.rank, S.world, config.get("heap_bytes"), backend)
    except _lib.TorchMPIError:
        ok = False
    flags = [None] * S.world
    dist.all_gather_object(flags, ok)
    if not all(flags) and backend == 1:
        # some rank could not use the virtual-memory API: everybody falls back to cudaIpc
        if h is not None:
            h.destroy()
        h = CudaHeap(S.rank, S.world, config.get("heap_bytes"), 0)
    elif not all(flags):
        raise RuntimeError("could not create the CUDA symmetric heap: " + _lib.last_error())
    if S.world > 1:
        h.rendezvous()
    return h
