"""Builds the C-ABI library (libsparsebench_b200.so) in-tree with nvcc for sm_100a.

The library is plain CUDA C++ behind `extern "C"` entry points (include/sparsebench_b200.h); it
does not link against torch or libcuda. `build()` recompiles only when a source is newer than the
library, so importing code can call it freely.
"""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIB_PATH = PACKAGE_DIR / "libsparsebench_b200.so"
SOURCES = ["common.cu", "routing.cu", "combine.cu", "tensormap.cu", "sdd.cu", "dsd.cu", "assigned.cu", "router.cu", "ep.cu", "rounding.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--shared",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found: set NVCC or put it on PATH to build libsparsebench_b200.so")


def sources() -> list[Path]:
    return [CSRC_DIR / name for name in SOURCES if (CSRC_DIR / name).exists()]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "sparsebench_b200.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every CUDA source into one shared library. Returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB_PATH), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
