"""Runs a function as N ranks in N child processes (gloo on CPU, or one GPU per rank)."""
import multiprocessing as mp
import os
import queue
import socket
import sys
import time
import traceback


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(fn, rank, world, port, q, args, env):
    try:
        os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                           "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
        os.environ.update(env)
        res = fn(rank, world, *args)
        q.put((rank, "ok", res))
    except BaseException:  # noqa: BLE001 - report everything to the parent
        q.put((rank, "error", traceback.format_exc()))
        sys.exit(1)


def run_ranks(fn, world, *args, timeout=180, env=None):
    """Runs ``fn(rank, world, *args)`` in ``world`` spawned processes; returns the list of results.

    Raises with the child's traceback if any rank fails, and ends the children (by pid) on timeout.
    """
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args, env or {})) for r in range(world)]
    for p in procs:
        p.start()
    results, deadline = {}, time.time() + timeout
    try:
        while len(results) < world:
            left = deadline - time.time()
            if left <= 0:
                raise TimeoutError(f"ranks {sorted(set(range(world)) - set(results))} did not finish in {timeout}s")
            try:
                rank, status, payload = q.get(timeout=min(left, 1.0))
            except queue.Empty:
                dead = [i for i, p in enumerate(procs) if not p.is_alive() and i not in results]
                if dead and q.empty():
                    time.sleep(0.2)
                    if q.empty():
                        raise RuntimeError(f"rank(s) {dead} died without reporting (exit codes "
                                           f"{[procs[i].exitcode for i in dead]})")
                continue
            if status == "error":
                raise RuntimeError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10 if len(results) == world else 0.5)
            if p.is_alive():
                p.kill()
                p.join()
    return [results[r] for r in range(world)]
