"""The MoE layer forward pass with no host sync anywhere: the reference's sparsebench/moe.py surface.

    routing -> SDD + GELU -> DSD -> combine        (four kernel launches)

Every buffer is sized for the worst case on the host, so the CPU never waits for the GPU to learn
how many rows routing produced, and the whole call can be captured in a CUDA graph and replayed
with new tokens and new routing.
"""

from __future__ import annotations

from collections.abc import Callable

import torch

from sparsebench_b200.routing import route_device
from sparsebench_b200.spmm import combine, dsd, sdd

BLOCK_SIZE = 128


def _no_mark(stage: str) -> None:
    pass


def moe_forward(
    x: torch.Tensor,
    expert_idx: torch.Tensor,
    expert_weight: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    mark: Callable[[str], None] = _no_mark,
) -> torch.Tensor:
    """x [T, D], expert_idx / expert_weight [T, k], w1 [E, D, F], w2 [E, F, D] -> [T, D].
    bf16 weights and activations, fp32 accumulation inside the kernels
    (reference: sparsebench/moe.py:25-56).

    mark(stage) is called right after each stage is launched, with "routing",
    "SDD + GELU (fused)", "DSD", "combine" in that order; a per-stage benchmark records a CUDA
    event there."""
    num_experts, d_model, ffn_dim = w1.shape
    if w2.shape != (num_experts, ffn_dim, d_model):
        raise ValueError(f"w2 must be {(num_experts, ffn_dim, d_model)}, got {tuple(w2.shape)}")
    if x.shape[1] != d_model or expert_idx.shape != expert_weight.shape or expert_idx.shape[0] != x.shape[0]:
        raise ValueError("x must be [T, D] and expert_idx / expert_weight [T, k]")

    topo = route_device(expert_idx, num_experts, ffn_dim, BLOCK_SIZE)
    mark("routing")
    h = sdd(x, w1, topo, gelu=True)
    mark("SDD + GELU (fused)")
    y = dsd(h, w2.view(num_experts * ffn_dim, d_model), topo, version=5)
    mark("DSD")
    out = combine(y, expert_weight, topo)
    mark("combine")
    return out
