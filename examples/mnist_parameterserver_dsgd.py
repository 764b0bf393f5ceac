"""The parameter server used as a synchronous allreduce (mnist_parameterserver_dsgd.lua:62-88):
zero the server, barrier, everybody adds its gradient, barrier, everybody receives, divide by size."""
from common import SyntheticMNIST, accuracy, device_from_env
import torch
import torchmpi_b200 as mpi
from torchmpi_b200 import nn as mpinn, parameterserver as ps
from torchmpi_b200.models.mlp import logistic_regression

dev = device_from_env()
mpi.start(with_cuda=dev == "cuda")
net = logistic_regression().to(mpi.device)
mpinn.synchronize_parameters(net)
crit = torch.nn.NLLLoss()
params = list(net.parameters())
servers = [ps.init(torch.zeros_like(p)) for p in params]
for epoch in range(3):
    for s in SyntheticMNIST(mpi.rank(), mpi.size(), device=mpi.device):
        net.zero_grad()
        crit(net(s["input"]), s["target"]).backward()
        if mpi.rank() == 0:
            ps.sync_handles([ps.send(sv, p.grad, "zero") for sv, p in zip(servers, params)])
        mpi.barrier()
        ps.sync_handles([ps.send(sv, p.grad.contiguous(), "add") for sv, p in zip(servers, params)])
        mpi.barrier()
        ps.sync_handles([ps.receive(sv, p.grad) for sv, p in zip(servers, params)])
        mpi.barrier()
        with torch.no_grad():
            for p in params:
                p.add_(p.grad, alpha=-0.05 / mpi.size())
mpinn.check_with_allreduce(net)
if mpi.rank() == 0:
    print(f"accuracy {accuracy(net, SyntheticMNIST(device=mpi.device)):.3f}")
ps.free_all()
mpi.stop()
