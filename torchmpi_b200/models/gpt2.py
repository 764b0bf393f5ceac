"""GPT-2 decoder (medium: 24 layers, d = 1024, 16 heads, context 1024, vocabulary 50257).

Used by the hierarchical-training config: synchronous fused allreduce inside a group of GPUs, a
GPU-resident parameter server across groups.  The reference has no sequence model
(its largest network is a 6-layer Linear stack, test/async.lua:37-43).  With ``tc_linear=True`` the matrix
products of the MLP and projections go through ``ops.gemm.linear`` (the tcgen05 kernel), attention through
``ops.attention`` (its own tcgen05 forward kernel on the packed QKV projection; PyTorch's scaled-dot-product
attention otherwise, and for shapes that kernel does not take), layer norm through the one-pass ``ops.layernorm``
and the LM head through the pitched ``ops.gemm.wide_head``; the loss is ``ops.xent``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    n_layer: int = 24
    n_head: int = 16
    n_embd: int = 1024
    block_size: int = 1024
    vocab_size: int = 50257
    tc_linear: bool = False


def gpt2_medium(**kw) -> "GPT2":
    return GPT2(GPT2Config(**kw))


def gpt2_tiny(**kw) -> "GPT2":
    cfg = dict(n_layer=2, n_head=4, n_embd=128, block_size=64, vocab_size=512)
    cfg.update(kw)
    return GPT2(GPT2Config(**cfg))


class _Linear(nn.Linear):
    def __init__(self, i, o, tc, gelu=False):
        super().__init__(i, o)
        self.tc, self.gelu = tc, gelu

    def forward(self, x):
        if self.tc:
            from ..ops import gemm
            return gemm.linear(x, self.weight, self.bias, self.gelu)
        y = F.linear(x, self.weight, self.bias)
        return F.gelu(y) if self.gelu else y


def _layer_norm(c: "GPT2Config") -> nn.LayerNorm:
    if c.tc_linear:
        from ..ops.layernorm import LayerNorm
        return LayerNorm(c.n_embd)
    return nn.LayerNorm(c.n_embd)


class Block(nn.Module):
    def __init__(self, c: GPT2Config):
        super().__init__()
        self.n_head = c.n_head
        self.own_attention = c.tc_linear
        self.ln1 = _layer_norm(c)
        self.qkv = _Linear(c.n_embd, 3 * c.n_embd, c.tc_linear)
        self.proj = _Linear(c.n_embd, c.n_embd, c.tc_linear)
        self.ln2 = _layer_norm(c)
        self.fc = _Linear(c.n_embd, 4 * c.n_embd, c.tc_linear, gelu=True)
        self.out = _Linear(4 * c.n_embd, c.n_embd, c.tc_linear)

    def forward(self, x):
        B, T, C = x.shape
        qkv = self.qkv(self.ln1(x).to(x.dtype))
        if self.own_attention:
            from ..ops import attention
            a = attention.causal_attention(qkv, self.n_head)
        else:
            q, k, v = (t.view(B, T, self.n_head, C // self.n_head).transpose(1, 2) for t in qkv.split(C, dim=2))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
        x = x + self.proj(a)
        return x + self.out(self.fc(self.ln2(x).to(x.dtype)))


class GPT2(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.config = c = config
        self.wte = nn.Embedding(c.vocab_size, c.n_embd)
        self.wpe = nn.Embedding(c.block_size, c.n_embd)
        self.blocks = nn.ModuleList([Block(c) for _ in range(c.n_layer)])
        self.ln_f = _layer_norm(c)
        self.apply(self._init)
        for b in self.blocks:   # scaled init of the residual projections
            for lin in (b.proj, b.out):
                nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * c.n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        """Token ids [B, T] -> logits [B*T, vocab] (the embedding matrix is tied to the output layer)."""
        B, T = idx.shape
        pos = torch.arange(T, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        for b in self.blocks:
            x = b(x)
        x = self.ln_f(x).to(self.wte.weight.dtype)
        if self.config.tc_linear:
            from ..ops import gemm
            return gemm.wide_head(x.reshape(B * T, -1), self.wte.weight)      # [B*T, vocab] view of a pitched buffer
        return F.linear(x.view(B * T, -1), self.wte.weight)


class LMLoss(nn.Module):
    """Next-token cross-entropy over flattened logits; the fused kernel on CUDA.  ``unit_grad``: see
    ``ops.xent.cross_entropy`` (for training loops that call ``loss.backward()`` on this loss itself)."""

    def __init__(self, unit_grad: bool = False):
        super().__init__()
        self.unit_grad = unit_grad

    def forward(self, logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        from ..ops import xent
        return xent.cross_entropy(logits, targets.reshape(-1), self.unit_grad)
