"""Training loop shared by the Downpour / EASGD examples: local Nesterov momentum SGD plus a
parameter-server policy called once per step (examples/mnist/mnist_parameterserver_easgd.lua:61-94)."""
from common import SyntheticMNIST, accuracy
import torch
import torchmpi_b200 as mpi


def train(net, make_policy, epochs=5, lr=0.05, momentum=0.9, dp_level=None):
    crit = torch.nn.NLLLoss()
    policy = make_policy(net)
    bufs = [torch.zeros_like(p) for p in net.parameters()]
    step = 0
    data_rank, data_size = mpi.world_rank(), mpi.world_size()
    for epoch in range(epochs):
        for s in SyntheticMNIST(data_rank, data_size, device=mpi.device):
            step += 1
            net.zero_grad()
            crit(net(s["input"]), s["target"]).backward()
            if dp_level is not None:                   # synchronous allreduce inside the data-parallel group
                mpi.set_collective_span(dp_level, dp_level)
                from torchmpi_b200 import nn as mpinn
                mpinn.synchronize_gradients(net, scale=1.0 / len(mpi.intra_members(dp_level)))
            with torch.no_grad():                      # Nesterov momentum, applied locally
                for p, b in zip(net.parameters(), bufs):
                    b.mul_(momentum).add_(p.grad)
                    p.add_(p.grad + momentum * b, alpha=-lr)
            policy.update(step)
    return policy
