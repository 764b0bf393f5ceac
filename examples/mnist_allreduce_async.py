"""Data-parallel SGD with gradient allreduces overlapped with backward (mnist_allreduce_async.lua)."""
from common import SyntheticMNIST, accuracy, device_from_env
import torch
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn
from torchmpi_b200.engine import AllReduceSGDEngine
from torchmpi_b200.models.mlp import logistic_regression

dev = device_from_env()
mpi.start(with_cuda=dev == "cuda")
mpi.async_.init_streams(True)
net = logistic_regression().to(mpi.device)
ds = SyntheticMNIST(mpi.rank(), mpi.size(), device=mpi.device)
engine = AllReduceSGDEngine(usegpu=dev == "cuda", async_=True, fused=False, gradient_scale=1.0 / mpi.size())
engine.train(net, torch.nn.NLLLoss(), ds, lr=0.05, maxepoch=5)
mpinn.check_with_allreduce(net)
if mpi.rank() == 0:
    print(f"accuracy {accuracy(net, SyntheticMNIST(device=mpi.device)):.3f}")
mpi.stop()
