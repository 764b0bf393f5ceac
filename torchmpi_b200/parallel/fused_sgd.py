"""``FusedSGD``: bucketed gradient allreduce fused with the SGD step, overlapped with backward.

Parameters and gradients are re-homed into flat buckets inside the symmetric
heap.  An autograd hook notices when the last gradient of a bucket has been
produced and launches, on a high-priority side stream, ONE kernel for that bucket
(csrc/kernels/ar_sgd.cu): reduce this rank's shard of the gradients out of every
peer's memory, apply scale / weight decay / momentum to the fp32 master shard,
store the new working weights into every peer, clear the gradients.  Backward
keeps running on the compute stream meanwhile.  Optimizer state (fp32 master
weights, momentum) exists only for the shard a rank owns.

This is the data-parallel path of the reference - ``synchronizeGradients`` after
backward, or per-layer async allreduces, then torchnet's per-tensor update
(torchmpi/nn.lua:49-56,112-242; torchmpi/engine/sgdengine.lua:126-147) - folded
into one launch per bucket with no NCCL call and no elementwise kernel.

Several backward passes per step (gradient accumulation over micro-batches): run all but the last inside
``with opt.accumulate():``; those passes only add to the gradient buckets, and the buckets are reduced and applied
during the last pass, still overlapped with its backward.  All parameters of a bucket must share one dtype.
"""
from __future__ import annotations

import contextlib
from typing import Iterable, List, Optional, Sequence

import torch

from .. import config, runtime
from .._lib import SgdBucket, dtype_code
from ..runtime import S
from .flat_buckets import FlatBuckets, Bucket
from .symm_heap import LANE_OPT


class FusedSGD:
    def __init__(self, params: Iterable[torch.nn.Parameter], *, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False, grad_scale: float = 1.0,
                 master_weights: bool = True, bucket_bytes: Optional[int] = None, overlap: bool = True,
                 members: Optional[Sequence[int]] = None, algo: int = 0):
        if S.cuda_heap is None:
            raise RuntimeError("FusedSGD needs the CUDA symmetric heap (start(with_cuda=True))")
        self.heap = S.cuda_heap
        self.members = tuple(members) if members is not None else runtime.intra_members(runtime.collective_span()[0])
        self.N = len(self.members)
        self.me = self.members.index(S.rank)
        self.momentum, self.dampening, self.weight_decay, self.nesterov = momentum, dampening, weight_decay, nesterov
        self.grad_scale, self.algo, self.overlap = grad_scale, algo, overlap
        self.lr = 0.0
        self.step_count = 0
        self.launches = 0
        self._defer = False
        params = [p for p in params if p.requires_grad]
        self.buckets = FlatBuckets(params, bucket_bytes or config.get("bucket_bytes"), pad_to=128 * self.N,
                                   allocator=self.heap.allocator())
        dev = params[0].device
        for b in self.buckets.buckets:
            shard = b.numel // self.N
            low = b.weight.dtype != torch.float32
            b.extra["master"] = torch.empty(shard, dtype=torch.float32, device=dev) if (low and master_weights) else None
            b.extra["momentum"] = torch.zeros(shard, dtype=torch.float32, device=dev) if momentum != 0.0 else None
            b.extra["launched"] = False
        self.refresh_master()
        self.comm_stream = torch.cuda.Stream(priority=-1)
        self._hooks = self.buckets.register_ready_hooks(self._on_bucket_ready, pass_bucket=True) if overlap else []

    # ---- state
    def _shard(self, b: Bucket) -> slice:
        shard = b.numel // self.N
        return slice(self.me * shard, (self.me + 1) * shard)

    def refresh_master(self) -> None:
        """Copies this rank's shard of the working weights into the fp32 master (after a broadcast or load)."""
        for b in self.buckets.buckets:
            if b.extra["master"] is not None:
                b.extra["master"].copy_(b.weight[self._shard(b)])

    # ---- one step
    def begin_step(self, lr: float) -> None:
        self.lr = float(lr)
        for b in self.buckets.buckets:
            b.extra["launched"] = False

    def _launch(self, b: Bucket, stream: torch.cuda.Stream) -> None:
        sb = SgdBucket()
        sb.grad_off, sb.weight_off = b.grad_off, b.weight_off
        sb.master = b.extra["master"].data_ptr() if b.extra["master"] is not None else None
        sb.momentum = b.extra["momentum"].data_ptr() if b.extra["momentum"] is not None else None
        sb.n = b.numel
        sb.grad_dtype = sb.weight_dtype = dtype_code(b.weight.dtype)
        sb.lr, sb.momentum_coef, sb.dampening = self.lr, self.momentum, self.dampening
        sb.weight_decay, sb.grad_scale = self.weight_decay, self.grad_scale
        sb.nesterov, sb.first_step, sb.zero_grads = int(self.nesterov), int(self.step_count == 0), 1
        self.heap.allreduce_sgd(sb, self.members, algo=self.algo, stream=stream, lane=LANE_OPT)
        b.extra["launched"] = True
        self.launches += 1

    @contextlib.contextmanager
    def accumulate(self):
        """Backward passes inside this context add their gradients to the buckets without launching the reduction
        (micro-batches of one optimizer step); the next pass outside it reduces and applies the sum."""
        self._defer = True
        try:
            yield self
        finally:
            self._defer = False

    def _on_bucket_ready(self, b: Bucket) -> None:
        if self._defer:
            return
        # gradients of this bucket are complete on the compute stream: hand it to the comm stream
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        self._launch(b, self.comm_stream)

    def finish_step(self) -> None:
        """Launches the buckets no hook has launched (unused parameters, or overlap off) in bucket order,
        then makes the compute stream wait for the updated weights."""
        cur = torch.cuda.current_stream()
        pending = [b for b in self.buckets.buckets if not b.extra["launched"]]
        if pending:
            self.comm_stream.wait_stream(cur)
            for b in pending:
                b.pending = len(b.params)
                self._launch(b, self.comm_stream)
        cur.wait_stream(self.comm_stream)
        self.step_count += 1
        for b in self.buckets.buckets:
            b.extra["launched"] = False

    def step(self, lr: float) -> None:
        """Optimizer-style use with ``overlap=False``: call after ``loss.backward()``."""
        self.lr = float(lr)
        self.finish_step()

    def check(self) -> None:
        """Raises if a device-side wait of the optimizer lane gave up."""
        self.heap.check_status(LANE_OPT)

    # ---- checkpointing (collective over the optimizer's members: every one of them calls)
    def state_dict(self) -> dict:
        """Full (unsharded) fp32 master weights and momentum per bucket, gathered over the ranks that share this
        optimizer, with the layout that produced them (bucket lengths, group size, parameter offsets and sizes),
        so that a job with another group size or bucket size can still place every parameter's state."""
        out = {"step": self.step_count, "group_size": self.N, "buckets": []}
        for b in self.buckets.buckets:
            entry = {"numel": b.numel, "offsets": list(b.offsets), "sizes": [p.numel() for p in b.params]}
            for key in ("master", "momentum"):
                shard = b.extra[key]
                if shard is None:
                    entry[key] = None
                    continue
                full = torch.empty(b.numel, dtype=torch.float32, device=shard.device)
                if self.N > 1:
                    self.heap.allgatherv(shard, full, [shard.numel()] * self.N, self.members)
                    torch.cuda.current_stream().synchronize()
                else:
                    full.copy_(shard)
                entry[key] = full.cpu()
            out["buckets"].append(entry)
        return out

    def load_state_dict(self, state: dict) -> None:
        """Loads a ``state_dict``.  Same layout: this rank's shard is cut out of every bucket.  Another group size
        or bucket size: the state is re-placed parameter by parameter (the parameters and their order must be the
        same); anything else raises."""
        saved = state["buckets"]
        mine = self.buckets.buckets
        same = len(saved) == len(mine) and all(e.get("numel", b.numel) == b.numel for e, b in zip(saved, mine)) \
            and state.get("group_size", self.N) == self.N
        if same:
            for b, entry in zip(mine, saved):
                for key in ("master", "momentum"):
                    if b.extra[key] is not None and entry.get(key) is not None:
                        b.extra[key].copy_(entry[key][self._shard(b)])
            self.step_count = int(state["step"])
            return
        if any("sizes" not in e for e in saved):
            raise ValueError("optimizer state was saved with another bucket layout and carries no per-parameter "
                             "layout; it cannot be re-placed")
        old_sizes = [n for e in saved for n in e["sizes"]]
        new_sizes = [p.numel() for b in mine for p in b.params]
        if old_sizes != new_sizes:
            raise ValueError(f"optimizer state holds {len(old_sizes)} parameters of other sizes than this model's "
                             f"{len(new_sizes)}; refusing to load misaligned state")
        for key in ("master", "momentum"):
            pieces = []
            for e in saved:
                for off, n in zip(e["offsets"], e["sizes"]):
                    pieces.append(None if e.get(key) is None else e[key][off:off + n])
            it = iter(pieces)
            for b in mine:
                if b.extra[key] is None:
                    for _ in b.params:
                        next(it)
                    continue
                full = torch.zeros(b.numel, dtype=torch.float32)
                for off, p in zip(b.offsets, b.params):
                    piece = next(it)
                    if piece is not None:
                        full[off:off + p.numel()] = piece
                b.extra[key].copy_(full[self._shard(b)])
        self.step_count = int(state["step"])

    def remove_hooks(self) -> None:
        self.buckets.remove_hooks()
