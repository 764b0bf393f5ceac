"""Downpour SGD policy (reference: torchmpi/parameterserver/downpourupdate.lua).

Every step the gradients are added to a local accumulator; every
``send_frequency`` steps (first at ``init_delay + send_frequency``) the
accumulator is passed through ``local_update`` (for example ``lambda t:
t.mul_(-lr)``), added to the server, waited for, and cleared.  Integration
overwrites the local parameters with the fetched server values.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .update import Update


class DownpourUpdate(Update):
    def __init__(self, network, sharding_communicator: int = 0, dataparallel_communicator: int = 0,
                 update_frequency: int = 10, init_delay: int = 100, prefetch: int = 0,
                 send_frequency: int = 1, local_update: Optional[Callable] = None, debug: bool = False):
        super().__init__(network, sharding_communicator, dataparallel_communicator, update_frequency,
                         init_delay, prefetch, debug)
        self.send_frequency = send_frequency
        self.next_send = self.init_delay + self.send_frequency
        self.local_update = local_update
        self.accumulators: List[torch.Tensor] = []

    def _accumulate(self, grads) -> None:
        from ..ops import elementwise
        if not self.accumulators:
            self.accumulators = [torch.zeros_like(g) for g in grads]
        for a, g in zip(self.accumulators, grads):
            elementwise.downpour_accum(a, g)

    def _send(self, step: int) -> None:
        from . import send_tensors, sync_handles
        with torch.no_grad():
            self._accumulate(self.grads())
        if step == self.next_send:
            self.handles_send = send_tensors(self.params(), self.accumulators, "add", self.local_update)
            self.handles_send = sync_handles(self.handles_send)
            for a in self.accumulators:
                a.zero_()
            self.next_send += self.send_frequency

    def _integrate(self, step: int) -> bool:
        if step != self.next_integration:
            return False
        from . import integrate_tensors, sync_handles
        self.handles_prefetch = sync_handles(self.handles_prefetch)
        integrate_tensors(self.params(), lambda fetched, t: t.copy_(fetched))
        self.next_integration += self.update_frequency
        return True
