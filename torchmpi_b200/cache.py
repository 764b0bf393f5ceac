"""References the library keeps on behalf of the user (reference: torchmpi/cache.lua).

Parameter-server objects, the prefetch and send staging tensors of the helper
layer and the handles of asynchronous backward passes are remembered here so
that they can be released together.  ``free_references_to_tensor`` works on the
tensor passed in; the reference loops over undefined locals there
(torchmpi/cache.lua:39-40).
"""
from __future__ import annotations

import torch

parameter_servers: dict = {}            # key(tensor) -> (tensor, ParameterServer)
prefetch_tensor_references: dict = {}   # key(tensor) -> prefetch clone
send_tensor_references: dict = {}       # key(tensor) -> staging tensor
tensor_references: dict = {}            # key(tensor) -> anything else kept alive
async_details = None                    # set by torchmpi_b200.nn


def key(t: torch.Tensor):
    """Identity of a tensor's memory: views of one parameter map to one entry."""
    return (t.data_ptr(), t.numel(), t.dtype)


def _same(a, b) -> bool:
    return a is b or (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor)
                      and a.data_ptr() == b.data_ptr() and a.numel() == b.numel())


def free_references_to_tensor(t: torch.Tensor) -> None:
    for table in (tensor_references, send_tensor_references, prefetch_tensor_references):
        for k in [k for k, v in table.items() if k == key(t) or _same(v, t)]:
            del table[k]
    for k in [k for k, (orig, _) in parameter_servers.items() if k == key(t) or _same(orig, t)]:
        _, ps = parameter_servers.pop(k)
        ps.free(collective=False)


def free_all_tensor_references() -> None:
    tensor_references.clear()
    for _, ps in list(parameter_servers.values()):
        ps.free(collective=False)
    parameter_servers.clear()
    send_tensor_references.clear()
    prefetch_tensor_references.clear()


def free_descriptors() -> None:
    """Peer mappings belong to the symmetric heap, not to tensors: nothing to release per tensor."""


freeReferencesToTensor, freeAllTensorReferences, freeDescriptors = (
    free_references_to_tensor, free_all_tensor_references, free_descriptors)
