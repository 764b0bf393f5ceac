"""Model-parallel Linear (examples/mnist/mnist_modelparallel.lua:30-60): every rank holds a slice of the
input features; outputs and input gradients are summed over the ranks."""
from common import SyntheticMNIST, accuracy, device_from_env
import torch
import torchmpi_b200 as mpi


class _SumOverRanks(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t):
        out = t.contiguous().clone()
        mpi.allreduce_tensor(out)
        return out

    @staticmethod
    def backward(ctx, g):
        return g                                      # d(sum_r y_r)/dy_r = 1: the same gradient everywhere


class MPLinear(torch.nn.Module):
    """Linear over a contiguous slice of the input features; the partial products are allreduced."""

    def __init__(self, inp, out):
        super().__init__()
        n, r = mpi.size(), mpi.rank()
        per = (inp + n - 1) // n
        self.lo, self.hi = r * per, min(inp, (r + 1) * per)
        self.lin = torch.nn.Linear(self.hi - self.lo, out, bias=(r == 0))    # one rank owns the bias

    def forward(self, x):
        return _SumOverRanks.apply(self.lin(x.flatten(1)[:, self.lo:self.hi]))


dev = device_from_env()
mpi.start(with_cuda=dev == "cuda")
torch.manual_seed(0)
net = torch.nn.Sequential(MPLinear(784, 10), torch.nn.LogSoftmax(dim=1)).to(mpi.device)
ds = SyntheticMNIST(device=mpi.device)                # every rank sees the same batches: the model is split, not the data
crit = torch.nn.NLLLoss()
for epoch in range(5):
    for s in ds:
        net.zero_grad()
        crit(net(s["input"]), s["target"]).backward()
        with torch.no_grad():
            for p in net.parameters():
                p.add_(p.grad, alpha=-0.05)
acc = accuracy(net, ds)            # the forward pass is collective: every rank evaluates
if mpi.rank() == 0:
    print(f"accuracy {acc:.3f}")
mpi.stop()
