"""``AllReduceSGDEngine``: data-parallel synchronous SGD with hooks.

The reference subclasses torchnet's SGDEngine and weaves MPI work into its hook
calls (torchmpi/engine/sgdengine.lua:19-150).  This engine keeps the same
options (``usegpu, async_, devicesync, dynamicnetwork, debug``), the same hook
names and the same ``state`` dictionary, and contains the small training loop
itself.  On GPUs its default path is *fused*: parameters and gradients live in
flat buckets inside the symmetric heap, and as soon as backward has produced a
bucket one kernel sums it over the peers' memory, applies scaling, momentum and
the weight update, and writes the new weights to every peer - no NCCL call and
no separate optimizer kernel.  ``fused=False`` (and every CPU run) takes the
reference's shape: ``synchronize_gradients`` then a per-tensor update.

Per sample:  onSample -> forward -> onForward -> criterion -> onForwardCriterion
-> zero grads -> criterion backward -> onBackwardCriterion -> network backward
-> gradient synchronisation -> onBackward -> update -> onUpdate.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Iterable, Optional

import torch

from . import collectives, nn as mpinn, runtime
from .runtime import S

HOOKS = ["onStart", "onStartEpoch", "onSample", "onForward", "onForwardCriterion", "onBackwardCriterion",
         "onBackward", "onUpdate", "onEndEpoch", "onEnd"]


class AllReduceSGDEngine:
    def __init__(self, usegpu: bool = False, async_: bool = False, devicesync: bool = True,
                 dynamicnetwork: bool = True, debug: bool = False, *, fused: Optional[bool] = None,
                 momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
                 nesterov: bool = False, gradient_scale: float = 1.0, master_weights: bool = True,
                 bucket_bytes: Optional[int] = None, **kw):
        if "async" in kw:  # the reference's option name is a Python keyword
            async_ = kw.pop("async")
        if kw:
            raise TypeError(f"unknown options {sorted(kw)}")
        self.usegpu, self.async_, self.devicesync = usegpu, async_, devicesync
        self.dynamicnetwork, self.debug = dynamicnetwork, debug
        self.fused = (usegpu and S.with_cuda) if fused is None else fused
        self.momentum, self.dampening, self.weight_decay, self.nesterov = momentum, dampening, weight_decay, nesterov
        self.gradient_scale = gradient_scale
        self.master_weights = master_weights
        self.bucket_bytes = bucket_bytes
        self.hooks: Dict[str, Callable] = {}
        self.registered = False
        self._opt = None           # FusedSGD when fused
        self._momentum_bufs = {}
        self._profiling = False

    # ---- hooks
    def hook(self, name: str, state) -> None:
        assert name in HOOKS, name
        self._mpi_hook(name, state)
        fn = self.hooks.get(name)
        if fn is not None:
            fn(state)

    def _device_sync(self) -> None:
        runtime.barrier()
        if self.usegpu and S.with_cuda:
            torch.cuda.synchronize()

    def _profile_window(self, name, state) -> None:
        """With NVPROF (or TORCHMPI_PROFILE) set, brackets iterations 3..8 with cudaProfilerStart/Stop."""
        if not (os.environ.get("NVPROF") or os.environ.get("TORCHMPI_PROFILE")) or not S.with_cuda:
            return
        if name == "onSample" and state["t"] == 3:
            self._device_sync()
            torch.cuda.profiler.start()
            self._profiling = True
        elif name == "onSample" and state["t"] == 8 and self._profiling:
            self._device_sync()
            torch.cuda.profiler.stop()
            self._profiling = False

    def _mpi_hook(self, name, state) -> None:
        self._profile_window(name, state)
        if name == "onSample":
            if self.async_ and not self.fused and not self.registered:
                mpinn.register_async_mpi_backward(state["network"], scale=self.gradient_scale)
                if isinstance(state["criterion"], torch.nn.Module):
                    mpinn.register_async_mpi_backward(state["criterion"], scale=self.gradient_scale)
                self.registered = not self.dynamicnetwork   # a dynamic network is re-examined every sample
            if self.devicesync:
                self._device_sync()
            if self.debug:
                mpinn.check_with_allreduce(state["network"])
        elif name == "onBackwardCriterion":
            if self.devicesync:
                self._device_sync()
            it = state.get("iterator")
            if hasattr(it, "prefetch"):
                it.prefetch()

    # ---- training
    def _setup(self, network, criterion):
        if self.fused:
            from .parallel.fused_sgd import FusedSGD
            self._opt = FusedSGD(network.parameters(), momentum=self.momentum, dampening=self.dampening,
                                 weight_decay=self.weight_decay, nesterov=self.nesterov,
                                 grad_scale=self.gradient_scale, master_weights=self.master_weights,
                                 bucket_bytes=self.bucket_bytes, overlap=True)
            network._tmpi_buckets = self._opt.buckets
        if len(runtime.intra_members(runtime.collective_span()[0])) > 1:
            # initial one-shot synchronisation of the parameters from rank 0
            mpinn.synchronize_parameters(network)
            if isinstance(criterion, torch.nn.Module):
                mpinn.synchronize_parameters(criterion)
        if self._opt is not None:
            self._opt.refresh_master()

    def _plain_update(self, params: Iterable[torch.nn.Parameter], lr: float) -> None:
        """w += -lr * g per tensor (torchnet's SGD step), with optional momentum / weight decay."""
        with torch.no_grad():
            for p in params:
                if p.grad is None:
                    continue
                g = p.grad
                if self.weight_decay:
                    g = g.add(p.data, alpha=self.weight_decay)
                if self.momentum:
                    buf = self._momentum_bufs.get(id(p))
                    if buf is None:
                        buf = self._momentum_bufs[id(p)] = g.detach().clone()
                    else:
                        buf.mul_(self.momentum).add_(g, alpha=1 - self.dampening)
                    g = g.add(buf, alpha=self.momentum) if self.nesterov else buf
                p.data.add_(g, alpha=-lr)

    def train_step(self, state, sample) -> torch.Tensor:
        """One sample: forward, loss, backward, gradient allreduce, update.  Returns the loss tensor."""
        network, criterion = state["network"], state["criterion"]
        state["sample"] = sample
        self.hook("onSample", state)
        inp, target = sample["input"], sample["target"]
        out = network(inp)
        state["output"] = out
        self.hook("onForward", state)
        loss = criterion(out, target)
        state["loss"] = loss
        self.hook("onForwardCriterion", state)
        if self._opt is not None:
            self._opt.begin_step(state["lr"])
        else:
            for p in network.parameters():
                p.grad = None if p.grad is None else p.grad.zero_()
        self.hook("onBackwardCriterion", state)
        loss.backward()
        if self._opt is not None:
            self._opt.finish_step()      # buckets launched from the hooks; this flushes and joins streams
            self.hook("onBackward", state)
        else:
            if len(runtime.intra_members(runtime.collective_span()[0])) > 1:
                if self.async_:
                    mpinn.async_.synchronize_gradients(network)
                else:
                    mpinn.synchronize_gradients(network, scale=self.gradient_scale)
            elif self.gradient_scale != 1.0:
                for p in network.parameters():
                    if p.grad is not None:
                        p.grad.mul_(self.gradient_scale)
            self.hook("onBackward", state)
            self._plain_update(network.parameters(), state["lr"])
            if isinstance(criterion, torch.nn.Module) and any(True for _ in criterion.parameters()):
                self._plain_update(criterion.parameters(), state["lrcriterion"])
        state["t"] += 1
        self.hook("onUpdate", state)
        return loss

    def train(self, network, criterion, iterator, lr: float, lrcriterion: Optional[float] = None,
              maxepoch: int = 1000, maxsteps: Optional[int] = None):
        state = {"network": network, "criterion": criterion, "iterator": iterator, "lr": lr,
                 "lrcriterion": lr if lrcriterion is None else lrcriterion, "maxepoch": maxepoch,
                 "sample": None, "epoch": 0, "t": 0, "training": True}
        self._setup(network, criterion)
        network.train()
        self.hook("onStart", state)
        done = False
        while state["epoch"] < maxepoch and not done:
            self.hook("onStartEpoch", state)
            for sample in iterator:
                self.train_step(state, sample)
                if maxsteps is not None and state["t"] >= maxsteps:
                    done = True
                    break
            state["epoch"] += 1
            self.hook("onEndEpoch", state)
        self.hook("onEnd", state)
        return state

    @torch.no_grad()
    def test(self, network, iterator, criterion=None):
        state = {"network": network, "criterion": criterion, "iterator": iterator, "sample": None,
                 "t": 0, "training": False, "epoch": 0, "lr": 0.0, "lrcriterion": 0.0}
        was_training = network.training
        network.eval()
        user = self.hooks
        fn = lambda n: user.get(n, lambda s: None)(state)  # plain hooks: no MPI work when testing
        fn("onStart")
        for sample in iterator:
            state["sample"] = sample
            fn("onSample")
            state["output"] = network(sample["input"])
            fn("onForward")
            if criterion is not None:
                state["loss"] = criterion(state["output"], sample["target"])
                fn("onForwardCriterion")
            state["t"] += 1
        fn("onEnd")
        network.train(was_training)
        return state
