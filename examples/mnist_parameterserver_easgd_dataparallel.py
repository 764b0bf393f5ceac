"""EASGD across groups, synchronous data parallelism inside each group
(examples/mnist/mnist_parameterserver_easgd_dataparallel.lua:28-35,67-91): a custom communicator
level groups the ranks; gradients are allreduced inside a group (communicator 1) while the group
roots exchange with the parameter server sharded over everybody (communicator 0)."""
from common import SyntheticMNIST, accuracy, device_from_env
from _ps_common import train
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn, parameterserver as ps
from torchmpi_b200.models.mlp import logistic_regression

GROUP = 2
dev = device_from_env()
mpi.start(with_cuda=dev == "cuda", custom_communicator_init=lambda: mpi.push_communicator(str(mpi.rank() // GROUP)))
mpi.set_communicator(0)
net = logistic_regression().to(mpi.device)
mpi.set_collective_span(0, 0)
mpinn.synchronize_parameters(net)
train(net, lambda n: ps.EASGDUpdate(n, sharding_communicator=0, dataparallel_communicator=1, beta=0.9,
                                    update_frequency=10, init_delay=20, prefetch=5), dp_level=1)
mpi.set_communicator(1)
mpinn.check_with_allreduce(net)                        # members of one group hold the same parameters
mpi.set_communicator(0)
if mpi.rank() == 0:
    print(f"accuracy {accuracy(net, SyntheticMNIST(device=mpi.device)):.3f}")
ps.free_all()
mpi.stop()
