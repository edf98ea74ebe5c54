"""Builds ``libcce_b200.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Run ``python -m cut_cross_entropy._build`` (or call :func:`build`).  nvcc
cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR.parent / "csrc"
LIB_PATH = PKG_DIR / "libcce_b200.so"
SOURCES = ["api.cu"]
HEADERS = ["engine.cuh", "engine_pair.cuh", "ptx.cuh", "ptx_pair.cuh", "small_kernels.cuh", "../../include/cce_b200.h", "../../include/cce_b200_testing.h"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or add the CUDA toolkit to PATH")
    return cand


def _host_compiler() -> list[str]:
    # a system g++ if present: nvcc needs a host compiler with its standard library set up
    for cand in ("/usr/bin/g++",):
        if Path(cand).exists():
            return ["--compiler-bindir", cand]
    return []


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any((CSRC_DIR / f).resolve().stat().st_mtime > built for f in SOURCES + HEADERS)


TRACE_LIB_PATH = PKG_DIR / "libcce_b200_trace.so"


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources.

    ``trace=True`` builds ``libcce_b200_trace.so`` instead, with the pipeline's wait-cycle counters
    compiled in (select it at run time with ``CCE_B200_LIB``).
    """
    if trace:
        return _compile(TRACE_LIB_PATH, ["-DCCE_TRACE=1"], verbose)
    if not force and not is_stale():
        return LIB_PATH
    return _compile(LIB_PATH, [], verbose)


def _compile(out: Path, defines: list[str], verbose: bool) -> Path:
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        *(["-Xptxas", "-v"] if verbose else []),
        *_host_compiler(),
        "-shared", "-Xcompiler", "-fPIC", *defines,
        "-o", str(out),
        *[str(CSRC_DIR / s) for s in SOURCES],
    ]  # fmt: skip
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr, file=sys.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
