"""``BlockSequential``: a Sequential regrouped into blocks with flat parameters.

Behaviour of the reference container (torchmpi/BlockSequential.lua):
the child modules are regrouped, in order, into about ``partitions`` blocks of
near-equal parameter count - a block is closed when the next module would take
it past ``ceil(total / partitions)``, which may yield ``partitions + 1`` blocks -
and each block's parameters and gradients are flattened into one contiguous
tensor.  ``backward_step`` runs the backward pass of exactly one block, last
block first, and hands back that block's flat parameter and gradient tensors so
that the caller can start their allreduce while the earlier blocks are still
being differentiated.

``torch.autograd`` has no per-module backward, so in *stepwise* mode ``forward``
cuts the graph between blocks (each block sees a detached input that requires
grad) and ``backward_step`` differentiates one cut at a time.  Outside stepwise
mode the container is an ordinary module and the flat gradient blocks are
filled by a normal ``loss.backward()``.

``BlockSequential.tensor_parallel`` builds the model-parallel flavour: a stack
of column-/row-split linear layers (see ``tensor_parallel.py``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .flat_buckets import FlatBuckets


class BlockSequential(nn.Sequential):
    def __init__(self, partitions: int, *modules: nn.Module):
        assert isinstance(partitions, int) and partitions > 0
        super().__init__(*modules)
        self.num_partitions = partitions
        self.stepwise = False
        self._blocks: Optional[List[nn.Sequential]] = None
        self._tmpi_buckets: Optional[FlatBuckets] = None
        self._step_number = 0
        self._cuts: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self._current_grad_output = None
        self._allocator = None

    # ---- partitioning
    def set_allocator(self, allocator) -> None:
        """Places the flat blocks in a symmetric heap (must be called before the first forward)."""
        self._allocator = allocator

    def is_partitioned(self) -> bool:
        return self._blocks is not None

    def _partition(self) -> None:
        if self._blocks is not None:
            raise RuntimeError("You can only call this function once.")
        mods = list(self.children())
        sizes = [sum(p.numel() for p in m.parameters()) for m in mods]
        per_split = math.ceil(sum(sizes) / self.num_partitions)
        blocks, cur, cur_size = [], [], 0

        def has_params(ms):
            return any(True for mm in ms for _ in mm.parameters())

        for m, sz in zip(mods, sizes):
            if cur_size + sz > per_split and has_params(cur):
                blocks.append(cur)
                cur, cur_size = [m], sz
            else:
                # a parameter-less run of modules stays glued to the block that follows
                # (the reference drops such a run, torchmpi/BlockSequential.lua:59-67)
                cur.append(m)
                cur_size += sz
        if cur:
            if has_params(cur) or not blocks:
                blocks.append(cur)
            else:
                blocks[-1] += cur
        self._blocks = [nn.Sequential(*b) for b in blocks]
        groups = [[p for p in blk.parameters() if p.requires_grad] for blk in self._blocks]
        if any(groups):
            self._tmpi_buckets = FlatBuckets([p for g in groups for p in g], groups=groups,
                                             allocator=self._allocator, pad_to=1, align_bytes=1)
        # re-register the blocks as the children, like `self.modules = blocks`
        for k in list(self._modules.keys()):
            del self._modules[k]
        for i, blk in enumerate(self._blocks):
            self.add_module(str(i), blk)

    def get_parameter_blocks(self):
        self._partition()
        return self.parameter_blocks()

    def parameter_blocks(self):
        if self._blocks is None:
            self._partition()
        if self._tmpi_buckets is None:
            return [], []
        return self._tmpi_buckets.weight_blocks(), self._tmpi_buckets.grad_blocks()

    def num_blocks(self) -> int:
        if self._blocks is None:
            self._partition()
        return len(self._blocks)

    # ---- forward / backward
    def forward(self, input):
        if self._blocks is None:
            self._partition()
        if not self.stepwise:
            x = input
            for blk in self._blocks:
                x = blk(x)
            return x
        self._cuts = []
        self._step_number = 0
        x = input
        for blk in self._blocks:
            xin = x.detach()
            if xin.dtype.is_floating_point:
                xin.requires_grad_(True)
            out = blk(xin)
            self._cuts.append((xin, out))
            x = out
        return x.detach()

    def backward_step(self, input, grad_output, scale: float = 1.0):
        """Backward of one block (last first).  Returns ``(grad_input, param_block, grad_block)``,
        and ``(None, None, None)`` once every block has been done (then the counter wraps)."""
        if self._blocks is None:
            raise RuntimeError("BlockSequential must be partitioned before backward_step")
        if not self._cuts:
            raise RuntimeError("backward_step needs a forward pass in stepwise mode")
        self._step_number += 1
        if self._step_number == 1:
            self._current_grad_output = grad_output
        elif self._step_number == len(self._blocks) + 1:
            self._step_number = 0
            return None, None, None
        idx = len(self._blocks) - self._step_number
        xin, out = self._cuts[idx]
        g = self._current_grad_output
        torch.autograd.backward(out, g * scale if scale != 1.0 else g)
        self._current_grad_output = xin.grad
        # index the flat blocks by the block's position among blocks that have parameters
        pb, gb = None, None
        if self._tmpi_buckets is not None:
            have = [i for i, blk in enumerate(self._blocks) if any(True for _ in blk.parameters())]
            if idx in have:
                k = have.index(idx)
                pb, gb = self._tmpi_buckets.buckets[k].weight, self._tmpi_buckets.buckets[k].grad
        return self._current_grad_output, pb, gb

    def backward(self, input, grad_output, scale: float = 1.0):
        """Runs every ``backward_step`` and returns the gradient with respect to ``input``."""
        res, g = None, grad_output
        while g is not None:
            res = g
            g, _, _ = self.backward_step(input, g, scale)
        return res

    def zero_grad_parameters(self) -> None:
        if self._blocks is None:
            raise RuntimeError("BlockSequential must be partitioned before zero_grad_parameters")
        if self._tmpi_buckets is not None:
            self._tmpi_buckets.zero_grad()

    def update_parameters(self, learning_rate: float) -> None:
        if self._blocks is None:
            raise RuntimeError("BlockSequential must be partitioned before update_parameters")
        if self._tmpi_buckets is not None:
            with torch.no_grad():
                for w, g in zip(*self.parameter_blocks()):
                    w.add_(g, alpha=-learning_rate)

    # ---- model-parallel flavour
    @staticmethod
    def tensor_parallel(*args, **kwargs):
        from .tensor_parallel import TensorParallelMLP
        return TensorParallelMLP(*args, **kwargs)

    # camelCase aliases
    backwardStep = backward_step
    parameterBlocks = parameter_blocks
    getParameterBlocks = get_parameter_blocks
    zeroGradParameters = zero_grad_parameters
    updateParameters = update_parameters
