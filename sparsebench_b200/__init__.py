"""sparsebench_b200: the sync-free block-sparse MoE forward path for NVIDIA B200 (sm_100a).

Drop-in for the reference's hot path: `moe_forward` plus the routing / SDD / DSD operator surface,
served by hand-written CUDA kernels behind a C ABI (include/sparsebench_b200.h). Importing the
package does not load the CUDA library; the first operator call does, and fails loudly if it is
missing. There is no CPU or PyTorch fallback.
"""

from sparsebench_b200.moe import moe_forward, moe_forward_assigned, moe_forward_from_logits
from sparsebench_b200.routing import DeviceTopology, build_topology_cuda, route, route_and_layout, route_device
from sparsebench_b200.rounding import DeviceAssignments, moe_forward_rounded, token_rounding
from sparsebench_b200.spmm import combine, dsd, sdd
from sparsebench_b200.topology import Topology

__all__ = [
    "DeviceAssignments",
    "DeviceTopology",
    "Topology",
    "build_topology_cuda",
    "combine",
    "dsd",
    "moe_forward",
    "moe_forward_assigned",
    "moe_forward_from_logits",
    "moe_forward_rounded",
    "route",
    "route_and_layout",
    "route_device",
    "sdd",
    "token_rounding",
]
__version__ = "0.1.0"
