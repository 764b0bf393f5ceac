"""Step-driven schedule of parameter-server traffic (reference: torchmpi/parameterserver/update.lua).

``update(step)`` is called once per training step:

* at ``step == init_delay`` the parameters are sharded onto the server;
* prefetches start at ``init_delay + update_frequency + prefetch`` and then every
  ``update_frequency`` steps; integrations happen at ``init_delay + update_frequency``
  and then every ``update_frequency`` steps;
* when the sharding communicator differs from the data-parallel one, only rank 0
  of each data-parallel group talks to the server; it then broadcasts the
  integrated parameters inside its group;
* the cursor always returns to communicator 0.

Subclasses provide ``_integrate(step) -> bool`` and ``_send(step)``.
"""
from __future__ import annotations

from typing import List

import torch

from .. import runtime, scalars
from .. import nn as mpinn


class Update:
    def __init__(self, network: torch.nn.Module, sharding_communicator: int = 0,
                 dataparallel_communicator: int = 0, update_frequency: int = 10,
                 init_delay: int = 100, prefetch: int = 0, debug: bool = False):
        assert 0 <= prefetch <= update_frequency, f"Prefetch must be in [0, {update_frequency}]"
        self.network = network
        self.sharding_communicator = sharding_communicator
        self.dataparallel_communicator = dataparallel_communicator
        self.init_delay, self.update_frequency, self.prefetch = init_delay, update_frequency, prefetch
        self.init_parameter_server = init_delay
        self.next_prefetch = init_delay + update_frequency + prefetch
        self.next_integration = init_delay + update_frequency
        self.handles_send: List = []
        self.handles_prefetch: List = []
        self.debug = debug
        self.on_parameters_changed = None    # optional callback after an integration changed the parameters

    def params(self) -> List[torch.Tensor]:
        blocks = mpinn._blocks(self.network)
        if blocks is not None:
            return list(blocks[0])
        return [p.data for p in self.network.parameters()]

    def grads(self) -> List[torch.Tensor]:
        blocks = mpinn._blocks(self.network)
        if blocks is not None:
            return list(blocks[1])
        return [p.grad for p in self.network.parameters()]

    def _shard(self, step: int) -> None:
        if step == self.init_parameter_server:
            from . import init_tensors
            runtime.set_communicator(self.sharding_communicator)
            init_tensors(self.params())

    def _fetch(self, step: int) -> None:
        if step == self.next_prefetch:
            from . import prefetch_tensors, sync_handles
            self.handles_send = sync_handles(self.handles_send)
            self.handles_prefetch = prefetch_tensors(self.params())
            self.next_prefetch += self.update_frequency

    def _integrate(self, step: int) -> bool:
        raise NotImplementedError("NYI: needs to be overridden")

    def _send(self, step: int) -> None:
        raise NotImplementedError("NYI: needs to be overridden")

    def update(self, step: int) -> None:
        self._shard(step)
        need_broadcast = 0
        runtime.set_communicator(self.dataparallel_communicator)
        if self.sharding_communicator == self.dataparallel_communicator:
            fetch_integrate = True
        else:
            fetch_integrate = runtime.rank() == 0
        runtime.set_communicator(self.sharding_communicator)
        if step >= self.init_parameter_server:
            if fetch_integrate:
                self._fetch(step)
                need_broadcast = 1 if self._integrate(step) else 0
            self._send(step)
        if self.sharding_communicator != self.dataparallel_communicator:
            runtime.set_communicator(self.dataparallel_communicator)
            need_broadcast = scalars.allreduce_double(float(need_broadcast))
            if need_broadcast > 0:
                # the group root integrated: hand its parameters to the rest of the group
                b, e = runtime.collective_span()
                runtime.set_collective_span(self.dataparallel_communicator, self.dataparallel_communicator)
                try:
                    mpinn.synchronize_parameters(self.network)
                finally:
                    runtime.set_collective_span(b, e)
                if self.debug:
                    mpinn.check_with_allreduce(self.network)
        if need_broadcast and self.on_parameters_changed is not None:
            self.on_parameters_changed()     # e.g. refresh fp32 master weights kept by a fused optimizer
        runtime.set_communicator(0)
