"""Tracing: NVTX ranges around collectives and a per-process ring buffer of (op, algo, bytes, microseconds).

The reference has no tracing API; it wraps whole ranks in ``nvprof`` from its launch script
(scripts/wrap.sh:63-68) and brackets engine iterations 3..8 with cudaProfilerStart/Stop
(torchmpi/engine/sgdengine.lua:38-63).  Here:

* ``trace.enable()`` turns recording on; the collective front end then times every call (CUDA events
  for GPU tensors - this synchronises, so it is a debugging mode) and appends a record to the ring
  buffer kept by the native runtime;
* ``trace.range(name)`` is an NVTX range (a no-op without CUDA) for external profilers;
* ``trace.dump(path)`` writes the records as JSON lines, one file per rank.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import json
import time
from typing import Iterator, List

import torch

from .._lib import lib


def enable(on: bool = True) -> None:
    lib.tmpi_trace_enable(1 if on else 0)


def enabled() -> bool:
    v = C.c_int64()
    lib.tmpi_get_tunable(b"trace", C.byref(v))
    return v.value != 0


def clear() -> None:
    lib.tmpi_trace_clear()


def record(op: str, algo: str, nbytes: int, us: float) -> None:
    lib.tmpi_trace_record(op.encode(), algo.encode(), int(nbytes), float(us))


def records() -> List[dict]:
    buf = C.create_string_buffer(1 << 20)
    n = lib.tmpi_trace_dump(buf, len(buf))
    return [json.loads(line) for line in buf.raw[:n].decode().splitlines() if line]


def dump(path: str) -> int:
    rows = records()
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    return len(rows)


@contextlib.contextmanager
def range(name: str) -> Iterator[None]:  # noqa: A001 - mirrors nvtx.range
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


@contextlib.contextmanager
def timed(op: str, algo: str, nbytes: int, cuda: bool) -> Iterator[None]:
    """Times the body (device time for CUDA work) and records it when tracing is on."""
    if not enabled():
        with range(op):
            yield
        return
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        with range(op):
            yield
        e1.record()
        e1.synchronize()
        record(op, algo, nbytes, e0.elapsed_time(e1) * 1e3)
    else:
        t0 = time.perf_counter()
        yield
        record(op, algo, nbytes, (time.perf_counter() - t0) * 1e6)
