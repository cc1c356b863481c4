"""TEST/BENCH INFRASTRUCTURE, not product: builds the reference's own CUDA extension for sm_100 so
that the reference's GPU kernels can serve as a second oracle and as a same-machine comparison row.

    python oracle/build_ref_ext.py [/path/to/reference]
    (default: $SPARSEBENCH_REFERENCE, a checkout named `reference` next to this repository, or the copy under
    baseline/_ref)

The reference's build system is not run. Its ten source files (csrc/bindings.cpp, smoke.cu,
routing.cu, dsd.cpp, dsd_v1..v5.cu, sdd.cu: the list in its setup.py:14-25) are compiled where
they lie by torch.utils.cpp_extension.load with the same flags (-O3 -std=c++17 -lineinfo) and
`-gencode arch=compute_100,code=sm_100` (plain mma.sync / cp.async / ldmatrix code is
forward-compatible; the reference itself targets sm_80 and sm_90a). Output: oracle/_ref/
sparsebench_ref_C.so, git-ignored. Nothing of the reference's sources is copied into the repository.

load_ref_ext() imports the built module (no compiling) or returns None with the reason.
"""

from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

OUT_DIR = Path(__file__).resolve().parent / "_ref"
NAME = "sparsebench_ref_C"
SOURCES = ["bindings.cpp", "smoke.cu", "routing.cu", "dsd.cpp", "dsd_v1.cu", "dsd_v2.cu", "dsd_v3.cu", "dsd_v4.cu",
           "dsd_v5.cu", "sdd.cu"]


def reference_csrc(arg: str | None = None) -> Path | None:
    root = Path(__file__).resolve().parent.parent
    named = [arg, os.environ.get("SPARSEBENCH_REFERENCE"), root.parent / "reference", root / "baseline" / "_ref"]
    candidates = [Path(c) / "csrc" for c in named if c]
    for c in candidates:
        if (c / "bindings.cpp").exists():
            return c
    return None


def build(arg: str | None = None, verbose: bool = True) -> Path:
    csrc = reference_csrc(arg)
    if csrc is None:
        raise SystemExit("no checkout of the reference found")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    from torch.utils.cpp_extension import load

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    load(name=NAME, sources=[str(csrc / s) for s in SOURCES], build_directory=str(OUT_DIR),
         extra_cflags=["-O3", "-std=c++17"], extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo"],
         is_python_module=False, verbose=verbose)
    return OUT_DIR / f"{NAME}.so"


def load_ref_ext():
    """(module, None) or (None, reason). Only loads a prebuilt file; needs a GPU at call time, not at import."""
    path = OUT_DIR / f"{NAME}.so"
    if not path.exists():
        return None, f"{path.name} has not been built (python oracle/build_ref_ext.py)"
    try:
        import torch  # noqa: F401  (the extension links against libtorch)

        spec = importlib.util.spec_from_file_location(NAME, path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        return module, None
    except Exception as exc:  # noqa: BLE001 - the caller reports the reason
        return None, f"{path.name} does not load: {exc!r}"


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
