"""`sparsebench`: the reference project's import name, served by sparsebench_b200.

Code written against the reference keeps working unchanged:

    from sparsebench import moe_forward            # or: from sparsebench.moe import moe_forward
    from sparsebench import _C                     # arch_probe, build_topology_cuda, sdd_cuda, dsd_cuda
    from sparsebench.routing import route_device, build_topology_cuda, DeviceTopology
    from sparsebench.spmm import sdd, dsd

Every name here forwards to the B200 implementation (hand-written sm_100a kernels behind the C ABI
in include/sparsebench_b200.h); nothing is computed in this package.

The reference also ships CPU-side helpers next to its operators (reference.py, topology.py's
build_topology, workloads.py, token_rounding.py, timing.py, baselines.py). They are not part of the
hot path and are not re-implemented here. Point SPARSEBENCH_REFERENCE_PY at a directory that holds
the reference's own copies of those modules and they become importable as sparsebench.<module>,
so that the reference's test-suite runs as it is against these kernels.
"""

import os as _os
from pathlib import Path as _Path

from sparsebench_b200 import moe_forward, moe_forward_assigned

__all__ = ["moe_forward", "moe_forward_assigned", "reference_py_dir"]
__version__ = "0.1.0"


def reference_py_dir() -> _Path | None:
    """Directory with the reference's own CPU-side modules, or None: SPARSEBENCH_REFERENCE_PY if
    set, else baseline/_ref/sparsebench_ref next to this package (where baseline/make_ref_copy.py
    puts them)."""
    named = _os.environ.get("SPARSEBENCH_REFERENCE_PY")
    candidates = [_Path(named)] if named else []
    candidates.append(_Path(__file__).resolve().parent.parent / "baseline" / "_ref" / "sparsebench_ref")
    for path in candidates:
        if (path / "reference.py").exists():
            return path
    return None


_ref_dir = reference_py_dir()
if _ref_dir is not None:
    # Modules this package does not define (reference, workloads, ...) resolve from the reference's
    # copy; the ones it does define (moe, routing, spmm, topology, _C) come first and win.
    __path__.append(str(_ref_dir))
