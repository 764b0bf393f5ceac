"""Shared pieces of the examples: a synthetic MNIST-shaped dataset split by rank and a small trainer.

The reference's examples train a logistic regressor on MNIST (examples/mnist/*.lua) with a global batch
of 336 split over the ranks (examples/mnist/makeiterator.lua:30,44-46).  There is no dataset on this
machine, so the images are seeded noise whose label is a fixed linear function of the pixels: the
task is learnable and every run is reproducible.
"""
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


class SyntheticMNIST:
    """``len(ds)`` batches of (images [B,1,28,28], labels [B]); rank r of n sees every n-th batch."""

    def __init__(self, rank=0, size=1, batches=60, global_batch=336, device="cpu", seed=0):
        g = torch.Generator().manual_seed(seed)
        self.teacher = torch.randn(784, 10, generator=g)
        self.batch = global_batch // size
        self.rank, self.size, self.batches, self.device, self.seed = rank, size, batches, device, seed

    def __len__(self):
        return self.batches

    def __iter__(self):
        for i in range(self.batches):
            g = torch.Generator().manual_seed(self.seed * 7919 + i * self.size + self.rank + 1)
            x = (torch.rand(self.batch, 1, 28, 28, generator=g) - 0.5) * 2      # centred pixels
            y = (x.flatten(1) @ self.teacher).argmax(1)
            yield {"input": x.to(self.device), "target": y.to(self.device)}


def device_from_env():
    return "cuda" if os.environ.get("EXAMPLE_DEVICE", "cpu") == "cuda" and torch.cuda.is_available() else "cpu"


def accuracy(net, ds):
    hit = tot = 0
    with torch.no_grad():
        for s in ds:
            hit += (net(s["input"]).argmax(1) == s["target"]).sum().item()
            tot += s["target"].numel()
    return hit / max(1, tot)
