"""Single-host launcher: ``python -m torchmpi_b200.launch --nproc N [options] script.py [args...]``.

Starts N ranks of ``script.py`` on this host, one per GPU (or N CPU ranks), the way the reference's
``scripts/wrap.sh`` + ``mpirun`` do (scripts/wrap.sh:15-88):

* exports ``RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT`` (rendezvous on 127.0.0.1);
* pins every rank to its own slice of the host's cores (``--no-affinity`` turns this off), the
  counterpart of the per-rank ``numactl --physcpubind`` slice;
* ``--log-to-file DIR`` sends each rank's output to ``DIR/rank_<r>.log``, otherwise only rank 0
  (and ranks that fail) print;
* ``--profile`` sets ``TORCHMPI_PROFILE=1`` so that the engine brackets iterations 3..8 with
  ``cudaProfilerStart/Stop`` for an external profiler.

If a rank exits with an error the others are terminated (by PID) and its exit code is returned.
``torch.distributed.run`` works just as well; this launcher only adds affinity and log handling.
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import tempfile
import time


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def core_slice(local_rank: int, nproc: int, cores=None):
    """Cores [begin, end) of this rank: the host's usable cores cut into nproc equal slices."""
    cores = sorted(os.sched_getaffinity(0)) if cores is None else list(cores)
    per = max(1, len(cores) // nproc)
    begin = (local_rank * per) % len(cores)
    return cores[begin:begin + per]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="torchmpi_b200.launch")
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--no-affinity", action="store_true")
    ap.add_argument("--log-to-file", default=None, metavar="DIR")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("-m", dest="module", action="store_true", help="treat the script as a module name")
    ap.add_argument("script")
    ap.add_argument("args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    port = a.master_port or _free_port()
    if a.log_to_file:
        os.makedirs(a.log_to_file, exist_ok=True)
    procs, logs = [], []
    for r in range(a.nproc):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(a.nproc),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        if a.profile:
            env["TORCHMPI_PROFILE"] = "1"
        cmd = [sys.executable] + (["-m", a.script] if a.module else [a.script]) + a.args
        out = None
        if a.log_to_file:
            out = open(os.path.join(a.log_to_file, f"rank_{r}.log"), "w")
        elif r != 0:
            out = tempfile.TemporaryFile()      # kept quiet unless the rank fails
        cores = None if a.no_affinity else core_slice(r, a.nproc)

        def pin(cores=cores):
            if cores:
                os.sched_setaffinity(0, cores)
        p = subprocess.Popen(cmd, env=env, stdout=out, stderr=subprocess.STDOUT if out is not None else None,
                             preexec_fn=pin if cores else None)
        procs.append(p)
        logs.append(out)
    rc = 0
    try:
        alive = set(range(a.nproc))
        while alive:
            for r in list(alive):
                code = procs[r].poll()
                if code is None:
                    continue
                alive.discard(r)
                if code != 0 and rc == 0:
                    rc = code
                    if logs[r] is not None and not a.log_to_file:
                        logs[r].seek(0)
                        sys.stderr.write(f"--- rank {r} failed ({code}):\n{logs[r].read().decode(errors='replace')}\n")
                    for q in alive:               # stop the survivors, by PID
                        procs[q].send_signal(signal.SIGTERM)
            time.sleep(0.05)
    except KeyboardInterrupt:
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        rc = 130
    finally:
        for p in procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()
        for f in logs:
            if f is not None:
                f.close()
    return rc


if __name__ == "__main__":
    sys.exit(main())
