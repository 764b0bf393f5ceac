"""The host runtime under ThreadSanitizer: csrc/runtime/{config,handles,communicator}.cpp are compiled with
-fsanitize=thread into a small driver that hammers tunables, pools, handles and the communicator stack from
many threads (csrc/tests/tsan_driver.cpp).  A data race would print a report and fail the run.  CPU only."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "torchmpi_b200" / "csrc"


def _cuda_home():
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and (Path(cand) / "include" / "cuda_runtime.h").exists():
            return Path(cand)
    return None


@pytest.mark.skipif(shutil.which("g++") is None or _cuda_home() is None, reason="needs g++ and the CUDA headers")
def test_host_runtime_is_race_free_under_thread_sanitizer(tmp_path):
    cuda = _cuda_home()
    exe = tmp_path / "tsan_driver"
    srcs = [CSRC / "tests" / "tsan_driver.cpp", CSRC / "runtime" / "config.cpp", CSRC / "runtime" / "handles.cpp",
            CSRC / "runtime" / "communicator.cpp"]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-fPIE", "-pie", "-I", str(CSRC / "include"),
           "-I", str(cuda / "include"), *map(str, srcs), "-o", str(exe), "-L", str(cuda / "lib64"), "-lcudart",
           "-lpthread", "-ldl", "-lrt", f"-Wl,-rpath,{cuda / 'lib64'}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66 report_signal_unsafe=0")
    run = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=300)
    assert "ThreadSanitizer" not in run.stderr, run.stderr[-4000:]
    assert run.returncode == 0, (run.returncode, run.stdout[-500:], run.stderr[-2000:])
    assert "ok" in run.stdout
