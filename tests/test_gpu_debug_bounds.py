"""The multi-rank kernels under the debug build (-DTMPI_DEBUG_BOUNDS): every peer load and store checks its
address against the mapped heaps, records the first violation in the status word and skips the access.  The
emulated collective suite (2, 4 and 8 ranks on one GPU) must run clean under it: a recorded violation
surfaces as an error of ``check_status``.  Stands in for compute-sanitizer on these kernels."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_emulated_collectives_run_clean_under_recording_bounds_checks():
    env = dict(os.environ, TORCHMPI_DEBUG_BOUNDS="1", PYTHONPATH=str(ROOT))
    flavour = subprocess.run([sys.executable, "-c",
                              "from torchmpi_b200._lib import lib; print(lib.tmpi_debug_bounds_build())"],
                             env=env, cwd=ROOT, capture_output=True, text=True, timeout=1200)
    assert flavour.returncode == 0, flavour.stderr[-2000:]
    assert flavour.stdout.strip().endswith("1"), "the child did not load the debug build"
    run = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider",
                          "tests/test_gpu_emulated_collectives.py", "-m", "gpu",
                          "-k", "allreduce_variants or rank_fill or broadcast or reduce_allgather or oneshot_slots or fused_allreduce_sgd"],
                         env=env, cwd=ROOT, capture_output=True, text=True, timeout=1200)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-1000:]
