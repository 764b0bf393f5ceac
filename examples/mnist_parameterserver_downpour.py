"""Downpour SGD (examples/mnist/mnist_parameterserver_downpour.lua): gradients are accumulated locally
and, scaled by -lr, added to the sharded server; parameters are re-read from the server periodically."""
from common import SyntheticMNIST, accuracy, device_from_env
from _ps_common import train
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn, parameterserver as ps
from torchmpi_b200.models.mlp import logistic_regression

dev = device_from_env()
mpi.start(with_cuda=dev == "cuda")
net = logistic_regression().to(mpi.device)
mpinn.synchronize_parameters(net)
train(net, lambda n: ps.DownpourUpdate(n, update_frequency=10, init_delay=20, prefetch=5, send_frequency=2,
                                       local_update=lambda t: t.mul_(-0.05 / mpi.size())), lr=0.05)
if mpi.rank() == 0:
    print(f"accuracy {accuracy(net, SyntheticMNIST(device=mpi.device)):.3f}")
ps.free_all()
mpi.stop()
