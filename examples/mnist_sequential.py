"""Single-process baseline (examples/mnist/mnist_sequential.lua): no communication at all."""
from common import SyntheticMNIST, accuracy
import torch
from torchmpi_b200.models.mlp import logistic_regression

net, crit = logistic_regression(), torch.nn.NLLLoss()
ds = SyntheticMNIST()
for epoch in range(5):
    for s in ds:
        net.zero_grad()
        crit(net(s["input"]), s["target"]).backward()
        with torch.no_grad():
            for p in net.parameters():
                p.add_(p.grad, alpha=-0.05)
print(f"accuracy {accuracy(net, ds):.3f}")
