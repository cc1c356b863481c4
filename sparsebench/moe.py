"""sparsebench.moe (reference: sparsebench/moe.py): moe_forward and moe_forward_assigned."""

from sparsebench_b200.moe import BLOCK_SIZE, moe_forward, moe_forward_assigned  # noqa: F401
