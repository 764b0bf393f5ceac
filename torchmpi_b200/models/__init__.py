"""Model zoo of the benchmarks: MLP / logistic regression, ResNet-50, GPT-2, tensor-parallel MLP."""
from __future__ import annotations

import torch
import torch.nn as nn


def to_bf16_mixed(model: nn.Module) -> nn.Module:
    """bf16 weights and activations for matrix-shaped layers; normalisation layers keep fp32
    parameters and statistics (they take bf16 activations)."""
    for m in model.modules():
        if isinstance(m, (nn.Conv2d, nn.Linear, nn.Embedding)):
            m.to(torch.bfloat16)
    return model
