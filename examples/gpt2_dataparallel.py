"""Data-parallel training of a small GPT-2 on a synthetic next-token task with ``AllReduceSGDEngine``.

    python -m torchmpi_b200.launch --nproc 2 examples/gpt2_dataparallel.py

The reference stops at MNIST networks; this example shows the same engine and gradient synchronisation on a sequence
model.  On CUDA (``EXAMPLE_DEVICE=cuda``) the model runs with ``tc_linear=True``: its matrix products, attention, layer
norm and loss are the package's own kernels (sequence length 128 so that the attention kernel applies) and the
optimizer is the fused allreduce + SGD; on CPU everything falls back to PyTorch and the gradients travel over gloo.
"""
from common import device_from_env
import torch
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn
from torchmpi_b200.engine import AllReduceSGDEngine
from torchmpi_b200.models import gpt2

dev = device_from_env()
cuda = dev == "cuda"
mpi.start(with_cuda=cuda)
torch.manual_seed(0)
T, V = (128, 64) if cuda else (32, 32)
net = gpt2.gpt2_tiny(n_layer=2, n_head=2, n_embd=128, block_size=T, vocab_size=V, tc_linear=cuda).to(mpi.device)
if cuda:
    net = net.to(torch.bfloat16)


def batches(seed, n, batch=8):
    """Arithmetic sequences modulo V with a per-sequence start and step: the next token is determined by the previous two."""
    g = torch.Generator().manual_seed(seed)
    for _ in range(n):
        start = torch.randint(0, V, (batch, 1), generator=g)
        step = torch.randint(1, 4, (batch, 1), generator=g)
        seq = (start + step * torch.arange(T + 1)) % V
        yield {"input": seq[:, :-1].to(mpi.device), "target": seq[:, 1:].to(mpi.device)}


def accuracy():
    net.eval()
    hit = tot = 0
    with torch.no_grad():
        for b in batches(999, 4):
            pred = net(b["input"])[:, :V].float().argmax(-1).view(b["target"].shape)
            hit += (pred[:, 2:] == b["target"][:, 2:]).sum().item()      # the first two positions cannot be known
            tot += b["target"][:, 2:].numel()
    net.train()
    return hit / tot


engine = AllReduceSGDEngine(usegpu=cuda, fused=cuda, momentum=0.9, gradient_scale=1.0 / mpi.size())
data = list(batches(100 + mpi.rank(), 60))
state = engine.train(net, gpt2.LMLoss(), data, lr=0.05, maxepoch=3)
mpinn.check_with_allreduce(net)                       # the replicas agree
acc = accuracy()
mpi.check_with_allreduce(acc, "accuracy")
if mpi.rank() == 0:
    print(f"accuracy {acc:.3f} after {state['t']} steps")
mpi.stop()
