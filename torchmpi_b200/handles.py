"""Handles of asynchronous operations.

``mpi.syncHandle(h)`` of the reference waits for an MPI request, a future or a
stream and frees the handle (lib/resources.cpp:1173-1242).  A ``Handle`` here
wraps any mix of: ids of the native registry (host task + CUDA event), work
objects of ``torch.distributed``, and Python finalisers that run after the wait
(for example the copy out of a staging buffer).
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Optional

import torch

from ._lib import lib, check


class Handle:
    __slots__ = ("ids", "works", "finalizers", "keep", "_done")

    def __init__(self, ids: Iterable[int] = (), works: Iterable = (), finalizers: Iterable[Callable] = (), keep=()):
        self.ids: List[int] = [i for i in ids if i]
        self.works = [w for w in works if w is not None]
        self.finalizers = list(finalizers)
        self.keep = keep          # tensors that must outlive the operation
        self._done = False

    def done(self) -> bool:
        if self._done:
            return True
        if any(lib.tmpi_handle_done(i) == 0 for i in self.ids):
            return False
        return all(w.is_completed() for w in self.works)

    def wait_stream(self, stream: Optional[torch.cuda.Stream] = None) -> "Handle":
        """Device-side wait: ``stream`` (default: current) waits for the GPU work; the host does not block."""
        s = stream if stream is not None else torch.cuda.current_stream()
        for i in self.ids:
            check(lib.tmpi_handle_stream_wait(i, s.cuda_stream))
        return self

    def wait(self, timeout_ms: int = -1) -> None:
        """Blocks the host until the operation is complete; frees the handle."""
        if self._done:
            return
        for i in self.ids:
            st = lib.tmpi_handle_wait(i, timeout_ms)
            if st == 3:        # TMPI_ERR_TIMEOUT: the peer or the request is gone; later calls must not wait again
                from . import watchdog
                from ._lib import last_error
                watchdog.poison("an asynchronous operation timed out: " + last_error())
            check(st)
        for w in self.works:
            w.wait()
        for f in self.finalizers:
            f()
        self.ids, self.works, self.finalizers, self.keep = [], [], [], ()
        self._done = True

    def merge(self, other: Optional["Handle"]) -> "Handle":
        if other is not None:
            self.ids += other.ids
            self.works += other.works
            self.finalizers += other.finalizers
            self.keep = (self.keep, other.keep)
        return self


def sync_handle(h: Optional[Handle]) -> None:
    """Waits for an asynchronous collective (``mpi.syncHandle``)."""
    if h is not None:
        h.wait()


def sync_handles(hs: Iterable[Optional[Handle]]) -> None:
    for h in hs:
        sync_handle(h)


def sync_all() -> None:
    """Drains every operation of the native pools (``syncAll`` of lib/resources.cpp:463-481)."""
    check(lib.tmpi_sync_all())
