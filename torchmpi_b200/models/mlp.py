"""Small dense models: the MNIST-sized MLP of the plumbing config and the reference's logistic regressor."""
from __future__ import annotations

import torch
import torch.nn as nn


class MLP(nn.Module):
    """784 -> hidden (ReLU) -> 10 with log-softmax output (pair with ``nn.NLLLoss``)."""

    def __init__(self, inp: int = 784, hidden: int = 100, out: int = 10):
        super().__init__()
        self.fc1 = nn.Linear(inp, hidden)
        self.fc2 = nn.Linear(hidden, out)

    def forward(self, x):
        x = x.flatten(1)
        return torch.log_softmax(self.fc2(torch.relu(self.fc1(x))), dim=1)


def logistic_regression(inp: int = 784, out: int = 10) -> nn.Module:
    """``nn.Linear(784, 10)`` + log-softmax, the model of examples/mnist/mnist_allreduce.lua:31."""
    return nn.Sequential(nn.Flatten(), nn.Linear(inp, out), nn.LogSoftmax(dim=1))


def linear_stack(depth: int = 6, width: int = 512) -> nn.Sequential:
    """The 6-layer Linear stack of the reference's async timing test (test/async.lua:37-43)."""
    return nn.Sequential(*[nn.Linear(width, width) for _ in range(depth)])
