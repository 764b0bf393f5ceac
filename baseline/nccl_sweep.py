"""Comparison baseline 1: the reference's NCCL call per tensor, restated with this box's NCCL.

The reference issues one ``ncclAllReduce / ncclBcast / ncclReduce`` per tensor on the user's stream
(lib/collectives_cuda.cpp:887-892,960-967,1046-1052).  This script runs the same sweep harness as
the product (``torchmpi_b200.tester``) with the ``nccl`` variant only, so both sides share sizes,
dtypes, timing method (CUDA events, max over ranks) and bandwidth formulas.

    python -m torch.distributed.run --nproc-per-node N baseline/nccl_sweep.py [tester options]
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from torchmpi_b200 import tester  # noqa: E402

if __name__ == "__main__":
    sys.argv += ["--variants", "nccl", "--benchmark"]
    tester.main()
