"""sparsebench.topology (reference: sparsebench/topology.py).

The hot path only needs the `Topology` data type. The reference's module also holds the CPU
construction of a layout (build_topology, bsr_to_dense, dense_to_bsr), which its tests use as ground
truth: when the reference's own copy of the module is available (see sparsebench.reference_py_dir)
it is loaded and re-exported whole, so the ground truth stays the reference's code; otherwise only
the data type is offered.
"""

import importlib.util as _util

from sparsebench import reference_py_dir as _reference_py_dir

_dir = _reference_py_dir()
if _dir is not None and (_dir / "topology.py").exists():
    _spec = _util.spec_from_file_location("sparsebench._reference_topology", _dir / "topology.py")
    _module = _util.module_from_spec(_spec)
    _spec.loader.exec_module(_module)
    globals().update({k: v for k, v in vars(_module).items() if not k.startswith("_")})
else:
    from sparsebench_b200.topology import Topology  # noqa: F401
