"""Drop-in proof: the reference's OWN test files, unmodified, run against this repository's kernels.

baseline/make_ref_copy.py puts a copy of the reference's tests/ and of its CPU-side ground-truth
modules under baseline/_ref/ (git-ignored). Each test below runs one of those files in a child
pytest whose `sparsebench` import resolves to this repository's package of that name, i.e. every
`_C.*`, `route_device`, `sdd`, `dsd`, `moe_forward` call in the reference's tests lands in
libsparsebench_b200. Nothing of the reference's tests is copied into this directory.

Skipped when the copy is absent. Cases the reference's files skip themselves (e.g. DSD v5 on block
size 64) stay skipped; a failure or error fails the test here and the child's report is printed.
"""

from __future__ import annotations

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

# GPU test files of the reference (tests/test_*.py) and the least number of cases that must pass
# in each: the count the file holds at the pinned reference revision minus its own skips.
FILES = {
    "test_smoke.py": 2,
    "test_routing.py": 263,
    "test_sdd.py": 23,
    "test_dsd.py": 900,
    "test_moe.py": 11,
    "test_token_rounding.py": 12,
}

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not (REF / "tests").exists(),
                                                  reason="no copy of the reference under baseline/_ref")]


def run_reference_file(name: str, timeout_s: int = 1500) -> tuple[int, dict[str, int], str]:
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    env["SPARSEBENCH_REFERENCE_PY"] = str(REF / "sparsebench_ref")
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", "-p", "no:cacheprovider", "--rootdir", str(REF), "-q", "-x",
         "--no-header", f"tests/{name}"],
        cwd=REF, env=env, capture_output=True, text=True, timeout=timeout_s)
    text = proc.stdout + proc.stderr
    counts = {kind: int(n) for n, kind in re.findall(r"(\d+) (passed|failed|skipped|error|errors)", text.splitlines()[-1] if text.strip() else "")}
    return proc.returncode, counts, text


@pytest.mark.parametrize("name", list(FILES))
def test_reference_file_passes_unmodified(name: str) -> None:
    if not (REF / "tests" / name).exists():
        pytest.skip(f"the reference copy has no tests/{name}")
    rc, counts, text = run_reference_file(name)
    report = "\n".join(text.splitlines()[-40:])
    assert rc == 0, f"the reference's tests/{name} does not pass against this library:\n{report}"
    assert counts.get("failed", 0) == 0 and counts.get("error", 0) + counts.get("errors", 0) == 0, report
    assert counts.get("passed", 0) >= FILES[name], f"only {counts} in tests/{name}:\n{report}"
    print(f"reference tests/{name}: {counts}")
