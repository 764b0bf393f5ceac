"""Collectives of the control plane over either kind of group.

A communicator that the whole world creates together gets ordinary ``torch.distributed`` process groups
(gloo, plus NCCL for GPU tensors).  A communicator that a sub-group splits on its own - only its members
call ``push_communicator``, as the reference allows (lib/c_api.h:42-47) - cannot: creating a process group
needs every rank of the job (or, with local synchronisation, hangs as soon as a rank creates a second
group out of step with its peers).  Such communicators get a ``LightGroup``: the same operations written
with tagged point-to-point messages of the world group.  They carry control traffic (scalars, counts,
barriers) and the gloo / CPU fallback; the data plane of the peer-memory backends does not go through here.
The functions below take either kind and mirror the ``torch.distributed`` calls this package uses.
"""
from __future__ import annotations

import zlib
from typing import List, Sequence

import torch
import torch.distributed as dist


class _Done:
    """A completed work object (what ``Handle`` expects of ``torch.distributed`` work)."""

    def wait(self):
        return True

    def is_completed(self):
        return True


class LightGroup:
    def __init__(self, members: Sequence[int], my_world_rank: int):
        self.members = tuple(members)
        self.me = self.members.index(my_world_rank)
        self.rank = my_world_rank
        self.tag = zlib.crc32(("g" + ".".join(map(str, self.members))).encode()) & 0x3FFFFF

    def size(self) -> int:
        return len(self.members)

    # ---- helpers: host copies of the payload, tagged messages on the world group
    @staticmethod
    def _host(t: torch.Tensor) -> torch.Tensor:
        return t.detach().cpu().contiguous() if t.is_cuda else t.detach().contiguous()

    def _send(self, t, dst):
        return dist.isend(t, dst, tag=self.tag)

    def _recv(self, t, src):
        return dist.irecv(t, src, tag=self.tag)

    # ---- operations (member order fixes the summation order: identical bits on all ranks)
    def all_reduce(self, t: torch.Tensor) -> None:
        h = self._host(t)
        root = self.members[0]
        if self.rank == root:
            parts = [torch.empty_like(h) for _ in self.members[1:]]
            for w in [self._recv(p, r) for p, r in zip(parts, self.members[1:])]:
                w.wait()
            acc = h.clone()
            for p in parts:
                acc += p
            for w in [self._send(acc, r) for r in self.members[1:]]:
                w.wait()
            h = acc
        else:
            self._send(h, root).wait()
            h = torch.empty_like(h)
            self._recv(h, root).wait()
        t.copy_(h.view_as(t))

    def broadcast(self, t: torch.Tensor, src: int) -> None:
        if self.rank == src:
            h = self._host(t)
            for w in [self._send(h, r) for r in self.members if r != src]:
                w.wait()
        else:
            h = torch.empty(t.shape, dtype=t.dtype)
            self._recv(h, src).wait()
            t.copy_(h)

    def reduce(self, t: torch.Tensor, dst: int) -> None:
        h = self._host(t)
        if self.rank == dst:
            acc = None
            parts = {r: (h if r == dst else torch.empty_like(h)) for r in self.members}
            for w in [self._recv(parts[r], r) for r in self.members if r != dst]:
                w.wait()
            for r in self.members:
                acc = parts[r].clone() if acc is None else acc + parts[r]
            t.copy_(acc.view_as(t))
        else:
            self._send(h, dst).wait()

    def all_gather(self, outs: List[torch.Tensor], t: torch.Tensor) -> None:
        h = self._host(t)
        bufs = [h if r == self.rank else torch.empty_like(h) for r in self.members]
        works = [self._send(h, r) for r in self.members if r != self.rank]
        works += [self._recv(b, r) for b, r in zip(bufs, self.members) if r != self.rank]
        for w in works:
            w.wait()
        for o, b in zip(outs, bufs):
            o.copy_(b.view_as(o))

    def sendrecv(self, send: torch.Tensor, recv: torch.Tensor, dst: int, src: int) -> None:
        hs = self._host(send)
        hr = torch.empty(recv.shape, dtype=recv.dtype)
        for w in (self._send(hs, dst), self._recv(hr, src)):
            w.wait()
        recv.copy_(hr)


def _light(g) -> bool:
    return isinstance(g, LightGroup)


def all_reduce(t, group, async_op=False):
    if _light(group):
        group.all_reduce(t)
        return _Done() if async_op else None
    return dist.all_reduce(t, group=group, async_op=async_op)


def broadcast(t, src, group, async_op=False):
    if _light(group):
        group.broadcast(t, src)
        return _Done() if async_op else None
    return dist.broadcast(t, src=src, group=group, async_op=async_op)


def reduce(t, dst, group, async_op=False):
    if _light(group):
        group.reduce(t, dst)
        return _Done() if async_op else None
    return dist.reduce(t, dst=dst, group=group, async_op=async_op)


def all_gather(outs, t, group):
    if _light(group):
        return group.all_gather(outs, t)
    return dist.all_gather(outs, t, group=group)


def reduce_scatter_tensor(out, inp, group):
    if _light(group):
        tmp = inp.clone()
        group.all_reduce(tmp)
        n = out.numel()
        out.copy_(tmp.view(-1)[group.me * n:(group.me + 1) * n].view_as(out))
        return None
    return dist.reduce_scatter_tensor(out, inp, group=group)


def sendrecv(send, recv, dst, src, group):
    """Sends ``send`` to world rank ``dst`` and receives ``recv`` from world rank ``src``."""
    if _light(group):
        return group.sendrecv(send, recv, dst, src)
    ops = [dist.P2POp(dist.isend, send, dst, group=group), dist.P2POp(dist.irecv, recv, src, group=group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
