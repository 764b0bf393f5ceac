"""Tensor collectives: broadcast, reduce, allreduce, sendreceive, allgather (+ reduce_scatter).

Front end of every collective: argument checks, the collective span (flat or
hierarchical composition), the choice of backend, sync or async.  It takes the
place of lib/collectives.cpp and lib/collectives_cuda.cpp of the reference.
Tensors must be contiguous; their shape is ignored (docs/collectives.md:14-23).
The reduction is always a sum, optionally times ``scale`` (fused into the GPU
kernels); ``scale=1`` reproduces the reference, which never divides
(torchmpi/nn.lua:49-56).

Backends:
  ``p2p``   own data plane - CUDA peer-memory kernels on GPU tensors, the shared
            memory heap on CPU tensors of ranks on one host
  ``nccl``  NCCL through torch.distributed (GPU tensors; the comparison baseline)
  ``gloo``  gloo through torch.distributed (CPU tensors; GPU tensors are staged)
  ``mpi``   the "stock library" entry of the reference: gloo on CPU, NCCL on GPU
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import gdist

from . import _lib, config, runtime
from ._lib import lib, check, dtype_code
from .handles import Handle
from .runtime import S
from .utils import trace as _trace

ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3, "ring": 4}


def _check_tensor(t: torch.Tensor, name: str = "tensor") -> torch.Tensor:
    """Validates ``t`` and returns a flat view of its memory.  Collectives ignore shape, so a dense
    channels-last tensor is as good as a contiguous one; anything with gaps is rejected, as the
    reference rejects non-contiguous tensors (lib/collectives.cpp:64-66)."""
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a tensor")
    dtype_code(t.dtype)
    if t.is_contiguous():
        return t.view(-1)
    if t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last):
        return t.permute(0, 2, 3, 1).reshape(-1)
    if t.dim() == 5 and t.is_contiguous(memory_format=torch.channels_last_3d):
        return t.permute(0, 2, 3, 4, 1).reshape(-1)
    raise ValueError(f"{name} must be contiguous")


def _me(members: Sequence[int]) -> int:
    try:
        return tuple(members).index(S.rank)
    except ValueError:
        raise RuntimeError(f"rank {S.rank} is not in communicator {tuple(members)}") from None


def _resolve_backend(t: torch.Tensor, backend: Optional[str], members: Sequence[int], op: str) -> str:
    if backend is None:
        from . import selector
        backend = selector.select(t, op)
    if backend == "mpi":
        backend = "nccl" if t.is_cuda else "gloo"
    if backend == "p2p":
        if t.is_cuda:
            if S.cuda_heap is None or not S.cuda_heap.covers(members):
                backend = "nccl"
        elif not (S.shm_ready and all(m in S.shm_ranks for m in members)):
            backend = "gloo"
    if backend == "nccl" and not t.is_cuda:
        raise ValueError("the nccl backend needs CUDA tensors")
    if backend not in ("p2p", "nccl", "gloo"):
        raise ValueError(f"unknown backend '{backend}'")
    return backend


def _scale_inplace(t: torch.Tensor, scale: float) -> None:
    if scale != 1.0:
        if t.dtype.is_floating_point:
            t.mul_(scale)
        else:
            t.copy_((t.double() * scale).to(t.dtype))


# ---------------------------------------------------------------- flat primitives
def _flat_allreduce(inp, out, members, backend, scale, algo, async_op) -> Optional[Handle]:
    members = tuple(members)
    n = inp.numel()
    if len(members) == 1 or n == 0:
        if out is not inp:
            out.copy_(inp)
        _scale_inplace(out, scale)
        return Handle() if async_op else None
    backend = _resolve_backend(inp, backend, members, "allreduce")
    me = _me(members)
    if backend == "p2p" and inp.is_cuda:
        return S.cuda_heap.allreduce(inp, out, members, scale=scale, algo=algo, async_op=async_op)
    if backend == "p2p":
        arr = _lib.int_array(members)
        args = (inp.data_ptr(), out.data_ptr(), n, dtype_code(inp.dtype), float(scale), arr, len(members), me, algo)
        if async_op:
            return Handle(ids=[lib.tmpi_shm_allreduce_async(*args)], keep=(inp, out, arr))
        check(lib.tmpi_shm_allreduce(*args))
        return None
    group = runtime.group_for(members)
    if backend == "gloo" and inp.is_cuda:
        host = inp.detach().cpu()
        work = gdist.all_reduce(host, group, async_op=True)

        def fin():
            _scale_inplace(host, scale)
            out.copy_(host)
        h = Handle(works=[work], finalizers=[fin], keep=(host,))
    else:
        if out is not inp:
            out.copy_(inp)
        work = gdist.all_reduce(out, group, async_op=True)
        h = Handle(works=[work], finalizers=[lambda: _scale_inplace(out, scale)], keep=(out,))
    if async_op:
        return h
    h.wait()
    return None


def _flat_broadcast(t, root, members, backend, async_op) -> Optional[Handle]:
    members = tuple(members)
    if len(members) == 1 or t.numel() == 0:
        return Handle() if async_op else None
    if not 0 <= root < len(members):
        raise ValueError(f"root {root} outside communicator of size {len(members)}")
    backend = _resolve_backend(t, backend, members, "broadcast")
    me = _me(members)
    if backend == "p2p" and t.is_cuda:
        return S.cuda_heap.broadcast(t, root, members, async_op=async_op)
    if backend == "p2p":
        arr = _lib.int_array(members)
        args = (t.data_ptr(), t.numel(), dtype_code(t.dtype), root, arr, len(members), me)
        if async_op:
            return Handle(ids=[lib.tmpi_shm_broadcast_async(*args)], keep=(t, arr))
        check(lib.tmpi_shm_broadcast(*args))
        return None
    group = runtime.group_for(members)
    if backend == "gloo" and t.is_cuda:
        host = t.detach().cpu()
        work = gdist.broadcast(host, members[root], group, async_op=True)
        h = Handle(works=[work], finalizers=[lambda: t.copy_(host)], keep=(host,))
    else:
        h = Handle(works=[gdist.broadcast(t, members[root], group, async_op=True)], keep=(t,))
    if async_op:
        return h
    h.wait()
    return None


def _flat_reduce(inp, out, root, members, backend, async_op) -> Optional[Handle]:
    members = tuple(members)
    if len(members) == 1 or inp.numel() == 0:
        if out is not inp:
            out.copy_(inp)
        return Handle() if async_op else None
    if not 0 <= root < len(members):
        raise ValueError(f"root {root} outside communicator of size {len(members)}")
    backend = _resolve_backend(inp, backend, members, "reduce")
    me = _me(members)
    if backend == "p2p" and inp.is_cuda:
        return S.cuda_heap.reduce(inp, out, root, members, async_op=async_op)
    if backend == "p2p":
        arr = _lib.int_array(members)
        check(lib.tmpi_shm_reduce(inp.data_ptr(), out.data_ptr(), inp.numel(), dtype_code(inp.dtype), root,
                                  arr, len(members), me))
        return Handle() if async_op else None
    group = runtime.group_for(members)
    # torch.distributed reduces in place and leaves non-root buffers undefined: work on a copy
    tmp = (inp.detach().cpu() if (backend == "gloo" and inp.is_cuda) else inp.clone())
    work = gdist.reduce(tmp, members[root], group, async_op=True)

    def fin():
        if me == root:
            out.copy_(tmp)
    h = Handle(works=[work], finalizers=[fin], keep=(tmp, out))
    if async_op:
        return h
    h.wait()
    return None


# ---------------------------------------------------------------- span composition
def _span_plan():
    """('flat', members) or ('hier', inner, inter, cartesian) for the current collective span."""
    cached = runtime.plan_cache.get("span_plan")
    if cached is not None:
        return cached
    b, e = runtime.collective_span()
    outer = runtime.intra_members(b)
    if b == e or not config.get("use_hierarchical_collectives"):
        plan = ("flat", outer)
    else:
        inner = runtime.intra_members(e)
        inter = runtime.inter_members(e)
        if len(inner) == len(outer) or (len(inter) <= 1 and runtime.is_cartesian_communicator(e)):
            plan = ("flat", outer if len(inner) == len(outer) else inner)
        else:
            plan = ("hier", inner, inter, runtime.is_cartesian_communicator(e))
    runtime.plan_cache["span_plan"] = plan        # dropped whenever communicators, span or tunables change
    return plan


def _wait(h):
    if h is not None:
        h.wait()


def allreduce_tensor(inp: torch.Tensor, out: Optional[torch.Tensor] = None, *, scale: float = 1.0,
                     backend: Optional[str] = None, algo: str = "auto", async_op: bool = False):
    """``out = scale * sum over ranks of inp`` on the collective span (``out`` defaults to ``inp``).

    With a hierarchical span the sum runs inside each inner group, then across
    groups (every rank on a cartesian level; only the group roots followed by a
    broadcast on a tree level), as lib/collectives_cuda.cpp:501-581 does.
    """
    runtime._require_started()
    same = out is None or out is inp
    inp = _check_tensor(inp, "input")
    out = inp if same else _check_tensor(out, "output")
    if out.numel() != inp.numel() or out.dtype != inp.dtype:
        raise ValueError("allreduce: input and output must have the same number of elements and dtype")
    a = ALGOS[algo] if isinstance(algo, str) else int(algo)
    plan = _span_plan()
    if plan[0] == "flat":
        if async_op or not _trace.enabled():
            return _flat_allreduce(inp, out, plan[1], backend, scale, a, async_op)
        with _trace.timed("allreduce", str(algo), inp.numel() * inp.element_size(), inp.is_cuda):
            return _flat_allreduce(inp, out, plan[1], backend, scale, a, False)
    _, inner, inter, cartesian = plan

    def stages(run):
        """The intra -> inter (-> broadcast) chain; ``run(thunk)`` executes one stage."""
        run(lambda asy: _flat_allreduce(inp, out, inner, backend, 1.0 if len(inter) > 1 or not cartesian else scale, a, asy))
        if cartesian:
            if len(inter) > 1:
                run(lambda asy: _flat_allreduce(out, out, inter, backend, scale, a, asy))
        else:
            if len(inter) > 1:
                run(lambda asy: _flat_allreduce(out, out, inter, backend, scale, a, asy))
            run(lambda asy: _flat_broadcast(out, 0, inner, backend, asy))

    if not async_op:
        stages(lambda thunk: _wait(thunk(False)))
        return None
    return _async_chain(inp, out, backend, inner, stages)


class _ThreadWork:
    """A chain of dependent stages run to completion on a helper thread; looks like a work object of
    ``torch.distributed`` to ``Handle`` (``wait`` / ``is_completed``)."""

    def __init__(self, fn):
        import threading
        self.error = None

        def body():
            try:
                fn()
            except BaseException as e:      # re-raised in wait()
                self.error = e
        self.thread = threading.Thread(target=body, daemon=True)
        self.thread.start()

    def is_completed(self) -> bool:
        return not self.thread.is_alive()

    def wait(self) -> None:
        self.thread.join()
        if self.error is not None:
            raise self.error


def _async_chain(inp, out, backend, inner, stages) -> Handle:
    """Asynchronous hierarchical allreduce: the whole chain is handed off and a live handle returned at once,
    as the reference does with its collective offload pool (lib/collectives_cuda.cpp:771-803,840-864).

    GPU tensors on the peer-memory backend: every stage is enqueued on the ordered asynchronous lane (one
    worker thread, one stream), so the stages run in order on the device with no host wait in between and
    the launch returns within microseconds.  Other backends: one helper thread runs the stages in order."""
    be = _resolve_backend(inp, backend, inner, "allreduce")
    on_lane = (be == "p2p" and inp.is_cuda and S.cuda_heap is not None
               and not S.cuda_heap._needs_staging(inp) and not S.cuda_heap._needs_staging(out))
    if on_lane:
        h = Handle()
        stages(lambda thunk: h.merge(thunk(True)))
        return h
    stream = torch.cuda.current_stream() if inp.is_cuda else None
    ready = stream.record_event() if stream is not None else None

    def run_all():
        if inp.is_cuda:
            torch.cuda.set_device(inp.device)
            side = torch.cuda.Stream(device=inp.device)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                stages(lambda thunk: _wait(thunk(False)))
            side.synchronize()
        else:
            stages(lambda thunk: _wait(thunk(False)))
    return Handle(works=[_ThreadWork(run_all)], keep=(inp, out))


def broadcast_tensor(root: int, t: torch.Tensor, *, backend: Optional[str] = None, async_op: bool = False):
    """Copies ``t`` of rank ``root`` (rank in the outer communicator of the span) to every rank, in place."""
    runtime._require_started()
    t = _check_tensor(t)
    b, _ = runtime.collective_span()
    if async_op or not _trace.enabled():
        return _flat_broadcast(t, int(root), runtime.intra_members(b), backend, async_op)
    with _trace.timed("broadcast", "auto", t.numel() * t.element_size(), t.is_cuda):
        return _flat_broadcast(t, int(root), runtime.intra_members(b), backend, False)


def reduce_tensor(root: int, inp: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                  backend: Optional[str] = None, async_op: bool = False):
    """Sum to ``root``; only root's ``out`` is written, ``inp`` is left untouched when ``out`` is given."""
    runtime._require_started()
    same = out is None or out is inp
    inp = _check_tensor(inp, "input")
    out = inp if same else _check_tensor(out, "output")
    b, _ = runtime.collective_span()
    outer = runtime.intra_members(b)
    plan = _span_plan()
    root = int(root)
    if plan[0] == "flat" or not 0 <= root < len(outer) or S.rank not in plan[1]:
        return _flat_reduce(inp, out, root, outer, backend, async_op)
    # hierarchical span: sum inside every inner group to the member that shares the root's position, then
    # across the groups to the root (cartesian); on a tree level the group roots hold the partial sums, the
    # root's group root collects them and hands the result on inside its group
    _, inner, inter, cartesian = plan
    root_world = outer[root]
    tmp = torch.empty_like(inp)
    if cartesian:
        pos = _position_in_group(root_world, b)
        _wait(_flat_reduce(inp, tmp, pos, inner, backend, False))
        if S.rank == inner[pos] and len(inter) > 1:
            _wait(_flat_reduce(tmp, out if S.rank == root_world else tmp, inter.index(root_world), inter, backend, False))
        elif S.rank == root_world:
            out.copy_(tmp)
    else:
        _wait(_flat_reduce(inp, tmp, 0, inner, backend, False))
        root_group = _group_of(root_world, b)
        if S.rank == inner[0] and len(inter) > 1:
            _wait(_flat_reduce(tmp, tmp, inter.index(root_group[0]), inter, backend, False))
        if root_world in inner and root_world != inner[0]:
            _wait(_flat_broadcast(tmp, 0, inner, backend, False))      # the group root passes the sum on to the root
        if S.rank == root_world:
            out.copy_(tmp)
    return Handle() if async_op else None


def _group_of(world_rank: int, outer_level: int) -> tuple:
    """Inner group (world ranks, in group order) of the span's inner level that contains ``world_rank``."""
    return runtime.group_of(runtime.collective_span()[1], world_rank)


def _position_in_group(world_rank: int, outer_level: int) -> int:
    return _group_of(world_rank, outer_level).index(world_rank)


def sendreceive_tensor(t: torch.Tensor, src: int, dst: int, *, backend: Optional[str] = None):
    """Sends ``t`` to rank ``dst`` and replaces it by what rank ``src`` sent (``MPI_Sendrecv_replace``).

    Stays on the library point-to-point path (NCCL for GPU tensors, gloo for CPU).
    """
    runtime._require_started()
    t = _check_tensor(t)
    b, _ = runtime.collective_span()
    members = runtime.intra_members(b)
    if len(members) == 1:
        return None
    me = _me(members)
    if src == me and dst == me:
        return None
    group = runtime.group_for(members)
    use_host = t.is_cuda and backend == "gloo"
    buf = t.detach().cpu() if use_host else t
    recv = torch.empty_like(buf)
    gdist.sendrecv(buf, recv, members[dst], members[src], group)
    t.copy_(recv)
    return None


def allgather_tensor(inp: torch.Tensor, out: torch.Tensor, *, backend: Optional[str] = None,
                     equal_counts: bool = False) -> torch.Tensor:
    """Rank-ordered concatenation of every rank's ``inp`` (element counts may differ per rank).

    ``out`` is resized when it is too small, as lib/collectives.cpp:253-286 does; the
    tensor holding the result is returned.  The per-rank counts are exchanged on the control plane
    (the reference does the same with an ``MPI_Allgather``, lib/collectives.cpp:219), which costs about
    0.1 ms; a caller that knows every rank contributes ``inp.numel()`` elements passes
    ``equal_counts=True`` and skips the exchange.
    """
    runtime._require_started()
    inp = _check_tensor(inp, "input")
    _check_tensor(out, "output")        # `out` may be resized below, so it stays as passed
    b, _ = runtime.collective_span()
    members = runtime.intra_members(b)
    N, me = len(members), _me(members)
    if N == 1:
        if out.numel() < inp.numel():
            out.resize_(inp.numel())
        out.view(-1)[:inp.numel()].copy_(inp.view(-1))
        return out
    group = runtime.group_for(members)
    if equal_counts:
        counts = [inp.numel()] * N
    else:
        counts_t = torch.zeros(N, dtype=torch.int64)
        counts_t[me] = inp.numel()
        gdist.all_reduce(counts_t, group)  # control plane (gloo)
        counts = counts_t.tolist()
    total = sum(counts)
    if out.numel() < total:
        out.resize_(total)
    flat = out.view(-1)
    be = _resolve_backend(inp, backend, members, "allgather")
    if be == "p2p" and inp.is_cuda:
        S.cuda_heap.allgatherv(inp, flat, counts, members)
    elif be == "p2p":
        arr = _lib.int_array(members)
        carr = (C.c_int64 * N)(*counts)
        check(lib.tmpi_shm_allgather(inp.data_ptr(), flat.data_ptr(), inp.numel(), carr, dtype_code(inp.dtype),
                                     arr, N, me))
    else:
        src = inp.detach().cpu() if (be == "gloo" and inp.is_cuda) else inp
        outs = [torch.empty(c, dtype=src.dtype, device=src.device) for c in counts]
        if len(set(counts)) == 1:
            gdist.all_gather(outs, src.view(-1), group)
        else:
            # unequal counts: pad to the largest
            m = max(counts)
            pad = torch.zeros(m, dtype=src.dtype, device=src.device)
            pad[:src.numel()] = src.view(-1)
            bufs = [torch.empty_like(pad) for _ in range(N)]
            gdist.all_gather(bufs, pad, group)
            outs = [bufs[k][:counts[k]] for k in range(N)]
        off = 0
        for k in range(N):
            flat[off:off + counts[k]].copy_(outs[k])
            off += counts[k]
    return out


def reduce_scatter_tensor(inp: torch.Tensor, out: torch.Tensor, *, scale: float = 1.0,
                          backend: Optional[str] = None):
    """``out`` (n elements) = scale * sum over ranks of the caller-rank's slice of ``inp`` (n * size elements)."""
    runtime._require_started()
    inp, out = _check_tensor(inp, "input"), _check_tensor(out, "output")
    b, _ = runtime.collective_span()
    members = runtime.intra_members(b)
    N, me = len(members), _me(members)
    if inp.numel() != out.numel() * N:
        raise ValueError("reduce_scatter: input must hold size * output elements")
    if N == 1:
        out.view(-1).copy_(inp.view(-1))
        _scale_inplace(out, scale)
        return None
    be = _resolve_backend(inp, backend, members, "reduce_scatter")
    if be == "p2p" and inp.is_cuda:
        S.cuda_heap.reduce_scatter(inp, out, members, scale=scale)
        return None
    group = runtime.group_for(members)
    if be == "nccl":
        gdist.reduce_scatter_tensor(out.view(-1), inp.view(-1), group)
        _scale_inplace(out, scale)
        return None
    tmp = inp.detach().cpu().clone() if inp.is_cuda else inp.clone()
    if S.shm_ready and not inp.is_cuda and be == "p2p":
        arr = _lib.int_array(members)
        check(lib.tmpi_shm_allreduce(tmp.data_ptr(), tmp.data_ptr(), tmp.numel(), dtype_code(tmp.dtype),
                                     float(scale), arr, N, me, 0))
    else:
        gdist.all_reduce(tmp, group)
        _scale_inplace(tmp, scale)
    n = out.numel()
    out.view(-1).copy_(tmp.view(-1)[me * n:(me + 1) * n])
    return None
