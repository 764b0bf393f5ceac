"""Tunables of the native runtime.

``set(name, value)`` / ``get(name)`` address the table of csrc/runtime/config.cpp.
The reference's setter and getter names (lib/c_api.h:96-152) exist as functions
of this module too; they must be called with the same value on every rank and
before the first collective, because pools and lanes are built lazily.
"""
from __future__ import annotations

import ctypes as C
import os

from ._lib import lib, check


def names() -> list:
    return [lib.tmpi_tunable_name(i).decode() for i in range(lib.tmpi_num_tunables())]


def set(name: str, value: int) -> None:  # noqa: A001 - mirrors the C API
    check(lib.tmpi_set_tunable(name.encode(), int(value)))
    from . import runtime
    runtime.plan_cache.clear()


def get(name: str) -> int:
    v = C.c_int64()
    check(lib.tmpi_get_tunable(name.encode(), C.byref(v)))
    return v.value


def freeze() -> None:
    check(lib.tmpi_freeze_tunables())


def as_dict() -> dict:
    return {n: get(n) for n in names()}


def load_env(prefix: str = "TORCHMPI_") -> None:
    """``TORCHMPI_<NAME>=<int>`` overrides a tunable (upper-cased name)."""
    for n in names():
        v = os.environ.get(prefix + n.upper())
        if v not in (None, ""):
            set(n, int(v))


def _pair(name: str):
    def setter(n: int) -> None:
        set(name, n)

    def getter() -> int:
        return get(name)
    setter.__name__, getter.__name__ = f"set_{name}", f"get_{name}"
    return setter, getter


for _n in ["small_cpu_broadcast_size", "small_cpu_allreduce_size", "small_gpu_broadcast_size",
           "small_gpu_allreduce_size", "min_buffer_size_per_cpu_collective",
           "min_buffer_size_per_gpu_collective", "max_buffer_size_per_cpu_collective",
           "max_buffer_size_per_gpu_collective", "num_buffers_per_cpu_collective",
           "num_buffers_per_gpu_collective", "collective_num_threads", "collective_thread_pool_size",
           "parameterserver_num_threads", "parameterserver_thread_pool_size",
           "broadcast_size_cpu_tree_based", "broadcast_size_gpu_tree_based"]:
    globals()[f"set_{_n}"], globals()[f"get_{_n}"] = _pair(_n)


def set_flat_collectives() -> None:
    set("use_hierarchical_collectives", 0)


def set_hierarchical_collectives() -> None:
    set("use_hierarchical_collectives", 1)


def set_staged_collectives() -> None:
    set("use_staged_collectives", 1)


def set_direct_collectives() -> None:
    set("use_staged_collectives", 0)


load_env()
