"""Which backend serves which collective.

The table has the reference's shape ``[cpu|gpu][singlenode|multinode][sync|async][collective]``
(torchmpi/init.lua:463-555) but its entries are backend names of this runtime.
GPU tensors default to the peer-memory kernels (``p2p``) whenever the symmetric
CUDA heap exists, with NCCL next; CPU tensors default to the shared-memory heap
on one host and to gloo across hosts.
"""
from __future__ import annotations

from typing import Optional

import torch

from .runtime import S

COLLECTIVES = ["allreduceTensor", "broadcastTensor", "reduceTensor", "sendreceiveTensor", "allgatherTensor"]
_OP_TO_NAME = {"allreduce": "allreduceTensor", "broadcast": "broadcastTensor", "reduce": "reduceTensor",
               "sendreceive": "sendreceiveTensor", "allgather": "allgatherTensor",
               "reduce_scatter": "allreduceTensor"}

collective_selector: Optional[dict] = None


def configure() -> None:
    """(Re)builds the table from what ``start`` found: heaps, NCCL, number of hosts."""
    global collective_selector
    has_nccl = S.with_cuda
    cpu_single = "p2p" if S.shm_ready else "gloo"
    gpu_p2p = "p2p" if (S.cuda_heap is not None and S.ipc_groups) else ("nccl" if has_nccl else "gloo")
    gpu_lib = "nccl" if has_nccl else "gloo"

    def table(dev: str, node: str) -> dict:
        if dev == "cpu":
            data = cpu_single if node == "singlenode" else "gloo"
            row = {"allreduceTensor": data, "broadcastTensor": data, "reduceTensor": data,
                   "sendreceiveTensor": "gloo", "allgatherTensor": data}
        else:
            data = gpu_p2p if node == "singlenode" else gpu_lib
            row = {"allreduceTensor": data, "broadcastTensor": data if S.single_ipc_group else gpu_lib,
                   "reduceTensor": data, "sendreceiveTensor": gpu_lib, "allgatherTensor": data}
        return {"sync": dict(row), "async": dict(row)}

    collective_selector = {d: {n: table(d, n) for n in ("singlenode", "multinode")} for d in ("cpu", "gpu")}


def select(t: torch.Tensor, op: str, mode: str = "sync") -> str:
    """Backend name for tensor ``t`` and collective ``op`` (tensor type -> cpu/gpu; hosts -> single/multi node)."""
    if collective_selector is None:
        configure()
    dev = "gpu" if t.is_cuda else "cpu"
    node = "multinode" if S.need_inter_node_collectives else "singlenode"
    return collective_selector[dev][node][mode][_OP_TO_NAME[op]]


def collective_selector_to_string(dev: Optional[str] = None, node: Optional[str] = None,
                                  mode: Optional[str] = None, coll: Optional[str] = None) -> str:
    assert dev in (None, "cpu", "gpu"), f"Invalid cpuSelector string {dev}"
    assert node in (None, "singlenode", "multinode"), f"Invalid nodeSelector string {node}"
    assert mode in (None, "sync", "async"), f"Invalid asyncSelector string {mode}"
    assert coll in (None, *COLLECTIVES), f"Invalid collectiveSelector string {coll}"
    if collective_selector is None:
        configure()
    out = []
    for c in ([dev] if dev else ["cpu", "gpu"]):
        for s in ([node] if node else ["singlenode", "multinode"]):
            for a in ([mode] if mode else ["sync", "async"]):
                for k in ([coll] if coll else COLLECTIVES):
                    be = collective_selector[c][s][a][k]
                    fn = "MPI." + ("async." if a == "async" else "") + ("" if be == "mpi" else be + ".") + k
                    out.append("MPI.collectiveSelector.%-40s \t->\t %s\n" % (f"{c}.{s}.{a}.{k}", fn))
    return "".join(out)


def collective_availability(cpu: bool = True, gpu: bool = True) -> Optional[str]:
    """One line per (device, sync/async, backend, collective): available / unimplemented / unavailable."""
    if collective_selector is None:
        return None
    lines = []
    for is_gpu in ([False] if cpu else []) + ([True] if gpu else []):
        lines.append("gpu = {\n" if is_gpu else "cpu = {\n")
        for is_async in (False, True):
            for be in ("", "nccl", "gloo", "p2p"):
                for coll in ("broadcast", "reduce", "allreduce", "sendreceive", "allgather"):
                    if be == "nccl" and not is_gpu:
                        continue
                    name = "MPI" + (".async" if is_async else "") + (f".{be}" if be else "") + f".{coll}Tensor"
                    val = "available"
                    if is_async and coll in ("sendreceive", "allgather"):
                        val = "unimplemented"
                    elif be == "nccl" and not S.with_cuda:
                        val = "unimplemented" if coll == "sendreceive" else "unavailable"
                    elif be == "p2p" and coll == "sendreceive":
                        val = "unimplemented"
                    elif be == "p2p" and is_gpu and S.cuda_heap is None:
                        val = "unavailable"
                    elif be == "p2p" and not is_gpu and not S.shm_ready:
                        val = "unavailable"
                    elif is_gpu and not S.with_cuda:
                        val = "unavailable"
                    lines.append("\t%-35s \t->\t %s\n" % (name, val))
        lines.append("}\n")
    return "".join(lines)
