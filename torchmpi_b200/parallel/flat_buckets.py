"""Flat parameter / gradient buckets.

Groups a model's parameters into a few contiguous blocks (weights in one flat
tensor, gradients in another), re-points every ``param.data`` / ``param.grad``
at a view of its block, and tells a callback when all gradients of a block have
been produced during backward.  One collective (or one fused
allreduce + optimizer kernel) then serves a whole block - the role of
``getParameters`` flattening in the reference's BlockSequential
(torchmpi/BlockSequential.lua:29-89), generalised to any module and placed in
the symmetric heap so that peer GPUs can read and write the blocks directly.
Blocks are filled in reverse parameter order: the gradients that backward
produces first share a block and can be reduced while the rest is computed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

ALIGN_BYTES = 128


@dataclass
class Bucket:
    index: int
    params: List[torch.nn.Parameter]
    offsets: List[int]                 # element offset of each param in the block
    numel: int                         # padded element count
    weight: torch.Tensor = None        # flat weights (model dtype)
    grad: torch.Tensor = None          # flat gradients (model dtype)
    weight_off: int = -1               # byte offsets inside the symmetric heap (-1: not in a heap)
    grad_off: int = -1
    pending: int = 0
    extra: dict = field(default_factory=dict)


def _dense(p: torch.Tensor) -> bool:
    return p.is_contiguous() or p.is_contiguous(memory_format=torch.channels_last) or \
        (p.dim() == 5 and p.is_contiguous(memory_format=torch.channels_last_3d))


class GradFork:
    """Sums the gradients that several consumers send into one activation without a separate add kernel.

    Autograd adds the gradients of a tensor that is used twice (the input of a residual block feeds the
    first convolution and the identity branch) with one more elementwise pass.  The consumers' backward
    functions can instead ``offer`` their gradient here: every consumer but the last parks its result and
    returns ``None`` to autograd; the last one computes ``its gradient + the parked sum`` in its own kernel
    (an epilogue that adds a tensor) and returns the total."""

    def __init__(self, consumers: int):
        self.consumers, self.seen, self.parked = consumers, 0, None

    def offer(self, make_grad):
        """``make_grad(add)`` returns this consumer's gradient, plus ``add`` when ``add`` is not None."""
        self.seen += 1
        g = make_grad(self.parked)
        if self.seen < self.consumers:
            self.parked = g
            return None
        self.seen, self.parked = 0, None
        return g


def direct_grad(param):
    """The gradient buffer that a backward kernel may add to in place of returning a gradient for ``param``
    (its view of a flat bucket whose readiness callback is installed), or None."""
    if param is None or getattr(param, "_tmpi_grad_sink", None) is None or param.grad is None:
        return None
    return param.grad


def grad_written(param) -> None:
    """Tells the bucket of ``param`` that its gradient has been added to ``param.grad`` in place.  Autograd may
    still run the parameter's post-accumulate hook afterwards although the backward function returned no
    gradient for it (it does in current PyTorch): that second report is recognised by the flag and dropped."""
    param._tmpi_reported = True
    param._tmpi_grad_sink(param, direct=True)


class FlatBuckets:
    def __init__(self, params: Sequence[torch.nn.Parameter], bucket_bytes: int = 32 << 20,
                 pad_to: int = 1024, allocator: Optional[Callable] = None, reverse: bool = True,
                 groups: Optional[Sequence[Sequence[torch.nn.Parameter]]] = None,
                 align_bytes: int = ALIGN_BYTES):
        """``allocator(nbytes) -> (uint8 tensor, heap byte offset)`` places blocks in a symmetric heap.

        ``groups`` fixes the partition (used by BlockSequential); otherwise parameters are packed
        greedily up to ``bucket_bytes``.  Every block's length is a multiple of ``pad_to`` elements
        so that it splits into equal, 16-byte aligned shards for any group size dividing ``pad_to``.
        """
        params = [p for p in params if p.requires_grad]
        if not params and not groups:
            raise ValueError("FlatBuckets: no trainable parameters")
        if groups is None:
            order = list(reversed(params)) if reverse else list(params)
            # one open block per (dtype, device): mixed-precision models (bf16 convolutions, fp32
            # batch-norm scales) still get a few large blocks instead of one per dtype switch
            groups, open_ = [], {}
            for p in order:
                nb = p.numel() * p.element_size()
                key = (p.dtype, p.device)
                cur = open_.get(key)
                if cur is not None and cur[1] + nb > bucket_bytes:
                    groups.append(cur[0])
                    cur = None
                if cur is None:
                    cur = open_[key] = [[], 0]
                cur[0].append(p)
                cur[1] += nb
            groups += [c[0] for c in open_.values() if c[0]]
        self.buckets: List[Bucket] = []
        self._hooks = []
        for gi, grp in enumerate(groups):
            grp = [p for p in grp if p.requires_grad]
            if not grp:
                continue
            dt, dev = grp[0].dtype, grp[0].device
            es = grp[0].element_size()
            align = max(1, align_bytes // es)
            offs, n = [], 0
            for p in grp:
                if p.dtype != dt or p.device != dev:
                    raise ValueError("FlatBuckets: parameters of one block must share dtype and device")
                offs.append(n)
                n += (p.numel() + align - 1) // align * align
            n = (n + pad_to - 1) // pad_to * pad_to
            b = Bucket(index=len(self.buckets), params=grp, offsets=offs, numel=n)
            b.weight, b.weight_off = self._alloc(n, dt, dev, allocator)
            b.grad, b.grad_off = self._alloc(n, dt, dev, allocator)
            b.weight.zero_()
            b.grad.zero_()
            for p, o in zip(grp, offs):
                wv = self._view(b.weight, o, p)
                gv = self._view(b.grad, o, p)
                with torch.no_grad():
                    wv.copy_(p.data)
                    if p.grad is not None:
                        gv.copy_(p.grad)
                p.data = wv
                p.grad = gv
            self.buckets.append(b)

    @staticmethod
    def _alloc(n, dt, dev, allocator):
        es = torch.empty((), dtype=dt).element_size()
        if allocator is not None and dev.type == "cuda":
            raw, off = allocator(n * es)
            return raw.view(dt)[:n], off
        return torch.empty(n, dtype=dt, device=dev), -1

    @staticmethod
    def _view(flat, off, p):
        seg = flat[off:off + p.numel()]
        if p.is_contiguous() or not _dense(p):
            return seg.view(p.shape)
        return seg.as_strided(p.shape, p.stride())   # keeps channels_last weights channels_last

    # ---- accessors
    def weight_blocks(self) -> List[torch.Tensor]:
        return [b.weight for b in self.buckets]

    def grad_blocks(self) -> List[torch.Tensor]:
        return [b.grad for b in self.buckets]

    def zero_grad(self) -> None:
        for b in self.buckets:
            b.grad.zero_()

    def repoint_grads(self) -> None:
        """Re-attaches ``param.grad`` views (after an optimizer or user code set them to None)."""
        for b in self.buckets:
            for p, o in zip(b.params, b.offsets):
                if p.grad is None or p.grad.data_ptr() != b.grad.data_ptr() + o * b.grad.element_size():
                    p.grad = self._view(b.grad, o, p)

    # ---- readiness hooks
    def register_ready_hooks(self, on_bucket: Callable[[torch.Tensor], None],
                             on_begin: Optional[Callable[[], None]] = None,
                             pass_bucket: bool = False) -> list:
        """``on_bucket(grad_block)`` (or ``on_bucket(bucket)``) runs inside backward as soon as every
        parameter of the block has its gradient; ``on_begin()`` runs at the first gradient of a pass."""
        handles = []
        for b in self.buckets:
            b.pending = len(b.params)
            for p in b.params:
                def hook(param, b=b, direct=False):
                    if not direct and getattr(param, "_tmpi_reported", False):
                        param._tmpi_reported = False      # already reported by the kernel that wrote the gradient
                        return
                    if on_begin is not None:
                        on_begin()
                    b.pending -= 1
                    if b.pending == 0:
                        b.pending = len(b.params)
                        on_bucket(b if pass_bucket else b.grad)
                handles.append(p.register_post_accumulate_grad_hook(hook))
                p._tmpi_grad_sink = hook      # kernels that add to p.grad in place call this instead (see direct_grad)
        self._hooks += handles
        return handles

    def remove_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for b in self.buckets:
            for p in b.params:
                if hasattr(p, "_tmpi_grad_sink"):
                    del p._tmpi_grad_sink
