"""Synchronous data-parallel SGD (examples/mnist/mnist_allreduce.lua).

    python -m torchmpi_b200.launch --nproc 4 examples/mnist_allreduce.py
"""
from common import SyntheticMNIST, accuracy, device_from_env
import torch
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn
from torchmpi_b200.engine import AllReduceSGDEngine
from torchmpi_b200.models.mlp import logistic_regression

dev = device_from_env()
mpi.start(with_cuda=dev == "cuda")
net = logistic_regression().to(mpi.device)
ds = SyntheticMNIST(mpi.rank(), mpi.size(), device=mpi.device)
engine = AllReduceSGDEngine(usegpu=dev == "cuda", fused=False, gradient_scale=1.0 / mpi.size())
state = engine.train(net, torch.nn.NLLLoss(), ds, lr=0.05, maxepoch=5)
mpinn.check_with_allreduce(net)                       # replicas agree at the end, as at the start
mpi.check_with_allreduce(accuracy(net, SyntheticMNIST(device=mpi.device)), "accuracy")
if mpi.rank() == 0:
    print(f"accuracy {accuracy(net, SyntheticMNIST(device=mpi.device)):.3f} after {state['t']} steps")
mpi.stop()
