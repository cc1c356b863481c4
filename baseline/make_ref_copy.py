"""Copies what the drop-in check needs from a checkout of the reference into baseline/_ref/.

    python baseline/make_ref_copy.py [/path/to/reference]        (default: /root/reference)

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

CPU_MODULES = ["reference.py", "topology.py", "workloads.py", "token_rounding.py", "timing.py", "baselines.py"]


def main() -> None:
    src = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference").resolve()
    dst = Path(__file__).resolve().parent / "_ref"
    if not (src / "sparsebench" / "reference.py").exists():
        raise SystemExit(f"{src} is not a checkout of the reference")
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


if __name__ == "__main__":
    main()
