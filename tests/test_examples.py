"""The examples run end to end as CPU ranks (the reference uses its MNIST scripts as integration tests,
scripts/test_cpu.sh:26-32)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
ENV = dict(os.environ, PYTHONPATH=str(ROOT), EXAMPLE_DEVICE="cpu")


def run(script, nproc):
    if nproc == 1:
        cmd = [sys.executable, str(ROOT / "examples" / script)]
    else:
        cmd = [sys.executable, "-m", "torchmpi_b200.launch", "--nproc", str(nproc), str(ROOT / "examples" / script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=ENV, cwd=str(ROOT / "examples"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("accuracy")][-1]
    return float(line.split()[1])


def test_sequential_baseline_learns():
    assert run("mnist_sequential.py", 1) > 0.5


@pytest.mark.parametrize("script,nproc", [("mnist_allreduce.py", 2), ("mnist_allreduce_async.py", 2),
                                          ("mnist_modelparallel.py", 2), ("mnist_parameterserver_dsgd.py", 2),
                                          ("mnist_parameterserver_downpour.py", 2),
                                          ("mnist_parameterserver_easgd.py", 2),
                                          ("mnist_parameterserver_easgd_dataparallel.py", 4),
                                          ("gpt2_dataparallel.py", 2)])
def test_distributed_examples(script, nproc):
    assert run(script, nproc) > 0.4


@pytest.mark.gpu
def test_gpt2_example_on_the_gpu_kernels():
    """One rank on a GPU: tcgen05 GEMMs and attention, fused layer norm, loss and allreduce + SGD."""
    env = dict(ENV, EXAMPLE_DEVICE="cuda")
    r = subprocess.run([sys.executable, str(ROOT / "examples" / "gpt2_dataparallel.py")], capture_output=True, text=True,
                       timeout=600, env=env, cwd=str(ROOT / "examples"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("accuracy")][-1]
    assert float(line.split()[1]) > 0.4
