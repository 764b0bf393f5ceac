"""Elastic-averaging SGD (examples/mnist/mnist_parameterserver_easgd.lua): every rank trains on its own
and is pulled towards a centre variable kept on the sharded server."""
from common import SyntheticMNIST, accuracy, device_from_env
from _ps_common import train
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn, parameterserver as ps
from torchmpi_b200.models.mlp import logistic_regression

dev = device_from_env()
mpi.start(with_cuda=dev == "cuda")
net = logistic_regression().to(mpi.device)
mpinn.synchronize_parameters(net)
train(net, lambda n: ps.EASGDUpdate(n, beta=0.9, update_frequency=10, init_delay=20, prefetch=5))
if mpi.rank() == 0:
    print(f"accuracy {accuracy(net, SyntheticMNIST(device=mpi.device)):.3f}")
ps.free_all()
mpi.stop()
