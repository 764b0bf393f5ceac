"""Elastic-averaging SGD policy (reference: torchmpi/parameterserver/easgdupdate.lua).

At each integration, with ``alpha = beta / size`` and ``c`` the fetched centre:
``d = c - x;  x += alpha * d;  delta = -alpha * d`` and ``delta`` is added to the
server, i.e. the centre moves by ``alpha * (x_old - c)``.  The reference stores
``delta`` keyed by tensor but sends by position, so nothing reaches the server
(torchmpi/parameterserver/easgdupdate.lua:49-50,66); here the deltas are kept in
parameter order and are sent.  On the GPU the three elementwise steps are one
kernel (``easgd_elastic``).
"""
from __future__ import annotations

from typing import List

import torch

from .. import cache, runtime
from .update import Update


class EASGDUpdate(Update):
    def __init__(self, network, sharding_communicator: int = 0, dataparallel_communicator: int = 0,
                 beta: float = 0.9, update_frequency: int = 10, init_delay: int = 100, prefetch: int = 0,
                 debug: bool = False):
        super().__init__(network, sharding_communicator, dataparallel_communicator, update_frequency,
                         init_delay, prefetch, debug)
        self.beta = beta
        self.next_send = self.next_integration
        self.deltas: List[torch.Tensor] = []
        self._have_deltas = False

    def _send(self, step: int) -> None:
        if step == self.next_send:
            if self._have_deltas:
                from . import send_tensors
                self.handles_send = send_tensors(self.params(), self.deltas, "add")
                self._have_deltas = False
            self.next_send += self.update_frequency

    def _integrate(self, step: int) -> bool:
        if step != self.next_integration:
            return False
        from . import integrate_tensors, sync_handles
        from ..ops import elementwise
        self.handles_prefetch = sync_handles(self.handles_prefetch)
        self.handles_send = sync_handles(self.handles_send)   # deltas are about to be overwritten
        alpha = self.beta / runtime.size()
        params = self.params()
        if not self.deltas:
            self.deltas = [torch.empty_like(p) for p in params]
        by_key = {cache.key(p): d for p, d in zip(params, self.deltas)}
        integrate_tensors(params, lambda fetched, t: elementwise.easgd_elastic(t, fetched, by_key[cache.key(t)], alpha))
        self._have_deltas = True
        self.next_integration += self.update_frequency
        return True
