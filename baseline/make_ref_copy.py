"""Copies what the drop-in check needs from a checkout of the reference into baseline/_ref/.

    python baseline/make_ref_copy.py [/path/to/reference]
    (default: $SPARSEBENCH_REFERENCE, else a checkout named `reference` next to this repository)

baseline/_ref/ is listed in .gitignore: the copy travels with the working tree to a GPU machine
but never enters the history. Laid out so that the reference's own `sparsebench` package is NOT
importable from it (the import name must resolve to this repository's package):

    baseline/_ref/tests/            the reference's tests/, byte for byte
    baseline/_ref/sparsebench_ref/  its CPU-side modules (ground truth of those tests):
                                    reference.py topology.py workloads.py token_rounding.py
                                    timing.py baselines.py
    baseline/_ref/csrc/             its CUDA sources, for oracle/build_ref_ext.py
"""

from __future__ import annotations

import shutil
import sys
from pathlib import Path

def find_reference(arg: str | None = None) -> Path | None:
    """A checkout of the reference: the argument, $SPARSEBENCH_REFERENCE, or ../reference beside the repository."""
    import os

    root = Path(__file__).resolve().parent.parent
    for candidate in (arg, os.environ.get("SPARSEBENCH_REFERENCE"), root.parent / "reference"):
        if candidate and (Path(candidate) / "sparsebench" / "reference.py").exists():
            return Path(candidate).resolve()
    return None


CPU_MODULES = ["reference.py", "topology.py", "workloads.py", "token_rounding.py", "timing.py", "baselines.py"]


def main(arg: str | None = None) -> Path:
    src = find_reference(arg)
    dst = Path(__file__).resolve().parent / "_ref"
    if src is None:
        raise SystemExit("no checkout of the reference found (argument, $SPARSEBENCH_REFERENCE or ../reference)")
    for name in ("tests", "sparsebench_ref", "csrc"):
        if (dst / name).exists():
            shutil.rmtree(dst / name)
    dst.mkdir(parents=True, exist_ok=True)
    shutil.copytree(src / "tests", dst / "tests", ignore=shutil.ignore_patterns("__pycache__"))
    (dst / "sparsebench_ref").mkdir()
    for name in CPU_MODULES:
        shutil.copy2(src / "sparsebench" / name, dst / "sparsebench_ref" / name)
    shutil.copytree(src / "csrc", dst / "csrc")
    print(f"copied tests/, {len(CPU_MODULES)} CPU modules and csrc/ from {src} to {dst}")
    return dst


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else None)
