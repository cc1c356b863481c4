"""The MoE layer forward pass with no host sync anywhere: the reference's sparsebench/moe.py surface.

    routing -> SDD + GELU -> DSD -> combine        (four kernel launches)

Every buffer is sized for the worst case on the host, so the CPU never waits for the GPU to learn
how many rows routing produced, and the whole call can be captured in a CUDA graph and replayed
with new tokens and new routing.
"""

from __future__ import annotations

import dataclasses
from collections.abc import Callable

import torch

from sparsebench_b200 import _C
from sparsebench_b200.routing import route_and_layout, route_device
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
    # Padding rows (up to 127 per expert) are neither stored by SDD nor read or stored by DSD in
    # whole groups of 32: nothing reads them, and H is the largest activation stream of the layer.
    h = sdd(x, w1, topo, gelu=True, skip_padding_rows=True, layout_from_routing=True)
    mark("SDD + GELU (fused)")
    y = dsd(h, w2.view(num_experts * ffn_dim, d_model), topo, version=5, skip_padding_rows=True,
            layout_from_routing=True)
    mark("DSD")
    out = combine(y, expert_weight, topo)
    mark("combine")
    return out


def moe_forward_from_logits(x: torch.Tensor, router_logits: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                            k: int = 2, mark: Callable[[str], None] = _no_mark, one_launch_routing: bool = False
                            ) -> torch.Tensor:
    """moe_forward with the router in front: router_logits [T, E] -> top-k experts and a softmax over the k
    picked logits (reference: sparsebench/reference.py:19-29), then the layer. Five launches; with
    one_launch_routing the router runs inside the routing kernel and the layer stays at four (slower as measured:
    see route_and_layout). The host never sees an expert id."""
    num_experts, d_model, ffn_dim = w1.shape
    if w2.shape != (num_experts, ffn_dim, d_model):
        raise ValueError(f"w2 must be {(num_experts, ffn_dim, d_model)}, got {tuple(w2.shape)}")
    if x.shape[1] != d_model or router_logits.shape != (x.shape[0], num_experts):
        raise ValueError("x must be [T, D] and router_logits [T, E]")
    _, expert_weight, topo = route_and_layout(router_logits, k, ffn_dim, BLOCK_SIZE, one_launch_routing)
    mark("routing")
    h = sdd(x, w1, topo, gelu=True, skip_padding_rows=True, layout_from_routing=True)
    mark("SDD + GELU (fused)")
    y = dsd(h, w2.view(num_experts * ffn_dim, d_model), topo, version=5, skip_padding_rows=True,
            layout_from_routing=True)
    mark("DSD")
    out = combine(y, expert_weight, topo)
    mark("combine")
    return out


def moe_forward_assigned(
    x: torch.Tensor,
    token_of_copy: torch.Tensor,
    expert_of_copy: torch.Tensor,
    weight_of_copy: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
) -> torch.Tensor:
    """The same layer for any routing given as a flat list: copy c sends token token_of_copy[c] to
    expert expert_of_copy[c] with weight weight_of_copy[c]. A token may have any number of copies,
    including none (its output row is 0), e.g. after a router that rounds per-expert counts
    (reference: sparsebench/moe.py:59-91).

    The copies go through routing as a k = 1 problem; the row -> copy table it leaves is turned into
    row -> token by one small kernel, SDD and DSD run unchanged, and the combine adds each copy's
    weighted row into its token in fp32. Still no host sync."""
    num_experts, d_model, ffn_dim = w1.shape
    num_tokens = x.shape[0]
    if expert_of_copy.numel() == 0:  # host-known size: nothing routed anywhere
        return torch.zeros_like(x)

    topo = route_device(expert_of_copy.reshape(-1, 1).contiguous(), num_experts, ffn_dim, BLOCK_SIZE)
    token_of_copy = token_of_copy.contiguous()
    # With k = 1 routing's row_token holds copy indices (-1 for padding): map them to tokens.
    topo = dataclasses.replace(topo, row_token=_C.remap_rows_cuda(topo.row_token, token_of_copy, num_tokens))
    h = sdd(x, w1, topo, gelu=True, skip_padding_rows=True, layout_from_routing=True)
    y = dsd(h, w2.view(num_experts * ffn_dim, d_model), topo, version=5, skip_padding_rows=True,
            layout_from_routing=True)
    return _C.combine_assigned_cuda(y, topo.copy_row, token_of_copy, weight_of_copy, num_tokens)
