"""Distributed helpers for ``torch.nn`` modules (reference: torchmpi/nn.lua).

``synchronize_parameters(net)``      broadcast every parameter from rank 0 (or average
                                     them with an allreduce)
``synchronize_gradients(net)``       sum every gradient over the ranks (``scale`` optional)
``check_with_allreduce(net)``        assert that parameters are replicated
``async_.register_async_mpi_backward(net)``  start each gradient's allreduce as soon as
                                     autograd has produced it, overlapped with the rest of
                                     backward; ``async_.synchronize_gradients`` then only waits.

A module that exposes flat blocks (``BlockSequential``, or any module holding a
``FlatBuckets`` in ``_tmpi_buckets``) is synchronised with one collective per
block instead of one per tensor.
"""
from __future__ import annotations

import types
from typing import List, Optional

import torch

from . import collectives, scalars, cache
from .handles import Handle
from .runtime import S


def _params(net) -> List[torch.nn.Parameter]:
    if isinstance(net, torch.nn.Module):
        return [p for p in net.parameters()]
    return list(net)


def _blocks(net):
    """Flat (parameter block, gradient block) tensors if the module has them, else None."""
    b = getattr(net, "_tmpi_buckets", None)
    if b is not None:
        return b.weight_blocks(), b.grad_blocks()
    if hasattr(net, "parameter_blocks") and getattr(net, "is_partitioned", lambda: False)():
        return net.parameter_blocks()
    return None


def synchronize_parameters(net, with_allreduce: bool = False) -> None:
    """Makes every rank hold rank 0's parameters (or, with ``with_allreduce``, their average)."""
    blocks = _blocks(net)
    tensors = blocks[0] if blocks is not None else [p.data for p in _params(net)]
    if isinstance(net, torch.nn.Module) and blocks is None:
        tensors = tensors + [b for b in net.buffers() if b.numel() > 0 and b.dtype.is_floating_point]
    b, _ = collectives.runtime.collective_span()
    world = len(collectives.runtime.intra_members(b))   # the span's outer communicator
    for w in tensors:
        if with_allreduce:
            collectives.allreduce_tensor(w, scale=1.0 / world)
        else:
            collectives.broadcast_tensor(0, w)


def synchronize_gradients(net, scale: float = 1.0) -> None:
    """In-place sum (times ``scale``) of every gradient over the ranks; no division by default,
    like torchmpi/nn.lua:49-56."""
    blocks = _blocks(net)
    if blocks is not None:
        for g in blocks[1]:
            collectives.allreduce_tensor(g, scale=scale)
        return
    for p in _params(net):
        if p.grad is not None:
            collectives.allreduce_tensor(p.grad, scale=scale)


def check_with_allreduce(net) -> None:
    if isinstance(net, torch.nn.Module):
        for name, p in net.named_parameters():
            scalars.check_with_allreduce(p.data, name)
    else:
        for i, p in enumerate(net):
            scalars.check_with_allreduce(p, str(i))


# ---------------------------------------------------------------- asynchronous flavour
class _AsyncState:
    def __init__(self):
        self.handles: List[Handle] = []
        self.counter = 0
        self.in_backward = False
        self.hooks = {}          # module id -> list of hook handles
        self.comm_stream: Optional[torch.cuda.Stream] = None


_A = _AsyncState()
cache.async_details = _A

skip_collective = set()   # modules whose gradients are left alone (declared, unused in the reference)


def _launch(grad: torch.Tensor, scale: float) -> None:
    """Async allreduce of one gradient tensor on the collective stream, after the compute stream."""
    if grad.is_cuda:
        if _A.comm_stream is None:
            _A.comm_stream = torch.cuda.Stream(priority=-1)
        cur = torch.cuda.current_stream()
        _A.comm_stream.wait_stream(cur)
        with torch.cuda.stream(_A.comm_stream):
            h = collectives.allreduce_tensor(grad, scale=scale, async_op=True)
    else:
        h = collectives.allreduce_tensor(grad, scale=scale, async_op=True)
    if h is not None:
        _A.handles.append(h)


def register_async_mpi_backward(net: torch.nn.Module, sync_gradient_frequency: int = 1, scale: float = 1.0) -> None:
    """After this call every backward pass starts the allreduce of a gradient the moment autograd
    has accumulated it.  With ``sync_gradient_frequency = k`` only every k-th backward pass
    communicates; the pass counter advances when a backward pass begins (the reference advances
    it in the first layer's backward, which runs last, torchmpi/nn.lua:137-144)."""
    if id(net) in _A.hooks:
        return
    hooks = []
    blocks = getattr(net, "_tmpi_buckets", None)

    def begin_pass():
        if not _A.in_backward:
            _A.in_backward = True
            _A.counter += 1

    if blocks is not None:
        hooks += blocks.register_ready_hooks(
            on_begin=begin_pass,
            on_bucket=lambda g: (_A.counter % sync_gradient_frequency == 0) and _launch(g, scale))
    else:
        for mod in net.modules():
            if mod in skip_collective:
                continue
            for p in mod.parameters(recurse=False):
                if not p.requires_grad:
                    continue

                def hook(param, _freq=sync_gradient_frequency):
                    begin_pass()
                    if _A.counter % _freq == 0 and param.grad is not None:
                        _launch(param.grad, scale)
                hooks.append(p.register_post_accumulate_grad_hook(hook))
    _A.hooks[id(net)] = hooks


def unregister_async_mpi_backward(net: torch.nn.Module) -> None:
    for h in _A.hooks.pop(id(net), []):
        h.remove()


def _async_synchronize_gradients(net=None) -> None:
    """Waits for the allreduces started during backward, newest first (torchmpi/nn.lua:207-212)."""
    for h in reversed(_A.handles):
        if S.with_cuda:
            h.wait_stream()
        h.wait()
    _A.handles = []
    _A.in_backward = False


async_ = types.SimpleNamespace(
    register_async_mpi_backward=register_async_mpi_backward,
    unregister_async_mpi_backward=unregister_async_mpi_backward,
    synchronize_gradients=_async_synchronize_gradients,
    skip_collective=skip_collective,
    registerAsyncMPIBackward=register_async_mpi_backward,
    unregisterAsyncMPIBackward=unregister_async_mpi_backward,
    synchronizeGradients=_async_synchronize_gradients,
    skipCollective=skip_collective,
)

synchronizeParameters, synchronizeGradients, checkWithAllreduce = (
    synchronize_parameters, synchronize_gradients, check_with_allreduce)
