"""Builds libtorchmpi_b200.so in-tree with nvcc for sm_100a.

``python -m torchmpi_b200.build`` compiles every file under ``csrc/runtime``
(host runtime) and ``csrc/kernels`` (CUDA) to an object under ``build/`` and
links them into ``torchmpi_b200/lib/libtorchmpi_b200.so``.  Objects are rebuilt
only when their source or a header is newer.  nvcc cross-compiles without a
GPU, so this runs on a CPU-only machine too.

The reference builds with CMake and an MPI compiler wrapper and knows no
architecture newer than Pascal (lib/CMakeLists.txt:1-94,
lib/cmake/select_compute_arch.cmake:20-36); here there is one architecture and
no optional dependency, so a short script replaces the CMake tree.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
# TORCHMPI_DEBUG_BOUNDS=1 selects the debug build: every peer load / store of the multi-rank kernels checks its
# address against the mapped heaps, records the first violation in the status word and skips the access
DEBUG_BOUNDS = bool(os.environ.get("TORCHMPI_DEBUG_BOUNDS"))
OBJ = PKG.parent / "build" / ("obj_dbg" if DEBUG_BOUNDS else "obj")
LIB = PKG / "lib" / ("libtorchmpi_b200_dbg.so" if DEBUG_BOUNDS else "libtorchmpi_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
          "--expt-relaxed-constexpr", "-I", str(CSRC / "include")]


def nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def sources() -> list[Path]:
    out = sorted((CSRC / "runtime").glob("*.cpp")) + sorted((CSRC / "runtime").glob("*.cu"))
    out += sorted((CSRC / "kernels").glob("*.cu"))
    return out


STAMP = PKG / "lib" / ("build_dbg.stamp" if DEBUG_BOUNDS else "build.stamp")


def source_hash() -> str:
    """Hash of every native source and header: the library is rebuilt when it changes."""
    import hashlib
    h = hashlib.sha256()
    for f in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + sources()):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def is_current() -> bool:
    return LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == source_hash()


def headers_mtime() -> float:
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(cc: str, src: Path, obj: Path, verbose: bool, extra: list[str]) -> tuple[Path, str]:
    cmd = [cc, *ARCH, *COMMON, *extra, "-x", "cu", "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return src, (r.stdout + r.stderr) if verbose else ""


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    cc = nvcc()
    if cc is None:
        raise RuntimeError("nvcc not found; cannot build libtorchmpi_b200.so")
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    import fcntl
    with open(OBJ.parent / "lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)     # ranks importing at the same time build once
        if not force and not ptxas_info and is_current():
            return LIB
        return _build_locked(cc, force, verbose, ptxas_info)


def _build_locked(cc: str, force: bool, verbose: bool, ptxas_info: bool) -> Path:
    hm = headers_mtime()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    if DEBUG_BOUNDS:
        extra.append("-DTMPI_DEBUG_BOUNDS")
    todo, objs = [], []
    for src in sources():
        obj = OBJ / (src.parent.name + "_" + src.stem + ".o")
        objs.append(obj)
        if force or ptxas_info or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hm):
            todo.append((src, obj))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            futs = [ex.submit(_compile, cc, s, o, verbose or ptxas_info, extra) for s, o in todo]
            for f in futs:
                src, log = f.result()
                if log:
                    print(f"--- {src.name}\n{log}", file=sys.stderr)
    if todo or not LIB.exists():
        cmd = [cc, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-lpthread", "-lrt", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    STAMP.write_text(source_hash())
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(p)
