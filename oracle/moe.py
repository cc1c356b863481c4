"""Floating-point side of the oracle: the MoE layer in plain CPU PyTorch.

TEST INFRASTRUCTURE (see oracle/__init__.py). Restates the reference's ground truth
(sparsebench/reference.py): expert e computes gelu(x @ w1[e]) @ w2[e] with the exact (erf) GELU,
each token takes the gate-weighted sum of its k experts' outputs. Works in whatever dtype it is
given (tests use fp32 on bf16-rounded values, or fp64).
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from oracle.layout import Layout, build_topology


def route(logits: torch.Tensor, k: int = 2) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k routing with a softmax over the k picked logits only, computed in fp32
    (reference: sparsebench/reference.py:19-29). Returns (expert_idx [T,k] int64, weight [T,k])."""
    if logits.dim() != 2 or not 0 < k <= logits.shape[1]:
        raise ValueError(f"need [T, E] logits with 0 < k <= E, got {tuple(logits.shape)} and k={k}")
    picked, expert_idx = torch.topk(logits, k, dim=-1)
    return expert_idx, torch.softmax(picked.float(), dim=-1).to(logits.dtype)


def check_shapes(x, expert_idx, expert_weight, w1, w2) -> None:
    """Same messages as the reference's _check_shapes (sparsebench/reference.py:32-46)."""
    if x.dim() != 2:
        raise ValueError(f"x must be [T, D], got {tuple(x.shape)}")
    num_tokens, d_model = x.shape
    if w1.dim() != 3 or w1.shape[1] != d_model:
        raise ValueError(f"w1 must be [E, {d_model}, F], got {tuple(w1.shape)}")
    num_experts, _, ffn_dim = w1.shape
    if w2.shape != (num_experts, ffn_dim, d_model):
        raise ValueError(f"w2 must be {(num_experts, ffn_dim, d_model)}, got {tuple(w2.shape)}")
    if expert_idx.dim() != 2 or expert_idx.shape[0] != num_tokens:
        raise ValueError(f"expert_idx must be [{num_tokens}, k], got {tuple(expert_idx.shape)}")
    if expert_weight.shape != expert_idx.shape:
        raise ValueError(f"expert_weight must match expert_idx shape {tuple(expert_idx.shape)}")


def moe_reference(x, expert_idx, expert_weight, w1, w2) -> torch.Tensor:
    """Loop over experts: gather the expert's tokens, run its MLP, scatter-add the gated result
    (reference: sparsebench/reference.py:49-61). x [T,D], idx/weight [T,k], w1 [E,D,F], w2 [E,F,D]."""
    check_shapes(x, expert_idx, expert_weight, w1, w2)
    out = torch.zeros_like(x)
    for e in range(w1.shape[0]):
        token, slot = torch.nonzero(expert_idx == e, as_tuple=True)
        if token.numel() == 0:
            continue
        y = F.gelu(x[token] @ w1[e]) @ w2[e]
        out.index_add_(0, token, y * expert_weight[token, slot, None])
    return out


def _gather_index(layout: Layout) -> tuple[torch.Tensor, torch.Tensor]:
    row_token = torch.from_numpy(layout.row_token.astype(np.int64))
    return row_token.clamp(min=0), row_token < 0


def group_tokens(x: torch.Tensor, layout: Layout) -> torch.Tensor:
    """[T, D] -> [P, D] in expert order, padding rows zero (reference: reference.py:82-87)."""
    index, is_padding = _gather_index(layout)
    grouped = x[index]
    grouped[is_padding] = 0
    return grouped


def sdd_blocks(x: torch.Tensor, w1: torch.Tensor, layout: Layout, gelu: bool) -> torch.Tensor:
    """Expected SDD output [nnz, bs, bs]: per row block, (gelu)(x_grouped @ w1[expert]) cut into
    bs-wide column blocks. Equal to the reference's dense product kept on the layout's blocks
    (reference.py:64-70 with tests/test_sdd.py:23-27) without forming the [P, E*F] matrix."""
    bs, fb = layout.block_size, layout.ffn_blocks
    grouped = group_tokens(x, layout)
    out = torch.zeros(layout.nnz_blocks, bs, bs, dtype=x.dtype)
    for rb in range(layout.num_row_blocks):
        e = int(layout.row_block_expert[rb])
        h = grouped[rb * bs : (rb + 1) * bs] @ w1[e]  # [bs, F]
        if gelu:
            h = F.gelu(h)
        begin = int(layout.row_offsets[rb])
        out[begin : begin + fb] = h.view(bs, fb, bs).permute(1, 0, 2)
    return out


def dsd_rows(blocks: torch.Tensor, w: torch.Tensor, layout: Layout) -> torch.Tensor:
    """Expected DSD output [P, D] for ANY BSR layout: row block r sums blocks[p] @ w[col_indices[p]
    * bs : +bs] over its p range (reference: reference.py:73-79; same definition as the
    reference test's bsr_matmul_oracle, tests/test_dsd.py:24-35)."""
    bs = layout.block_size
    out = torch.zeros(layout.num_row_blocks * bs, w.shape[1], dtype=blocks.dtype)
    for rb in range(layout.num_row_blocks):
        for p in range(int(layout.row_offsets[rb]), int(layout.row_offsets[rb + 1])):
            c = int(layout.col_indices[p])
            out[rb * bs : (rb + 1) * bs] += blocks[p] @ w[c * bs : (c + 1) * bs]
    return out


def ungroup_combine(y_rows: torch.Tensor, expert_weight: torch.Tensor, layout: Layout) -> torch.Tensor:
    """[P, D] -> [T, D]: each token's k rows, weighted and summed (reference: reference.py:90-94)."""
    num_tokens, k = expert_weight.shape
    rows = y_rows[torch.from_numpy(layout.copy_row.astype(np.int64))].view(num_tokens, k, -1)
    return (rows * expert_weight[..., None]).sum(dim=1)


def moe_blocksparse_reference(x, expert_idx, expert_weight, w1, w2, block_size: int) -> torch.Tensor:
    """The same layer through the block-sparse layout, stage by stage
    (reference: sparsebench/reference.py:97-114)."""
    check_shapes(x, expert_idx, expert_weight, w1, w2)
    num_experts, d_model, ffn_dim = w1.shape
    layout = build_topology(expert_idx, num_experts, ffn_dim, block_size)
    h = sdd_blocks(x, w1, layout, gelu=True)
    y_rows = dsd_rows(h, w2.reshape(num_experts * ffn_dim, d_model), layout)
    return ungroup_combine(y_rows, expert_weight, layout)


def moe_reference_streamed(x, expert_idx, expert_weight, w1, w2, dtype=torch.float32) -> torch.Tensor:
    """moe_reference for layers whose weights do not fit in memory as fp32: upcasts one expert at a
    time. Same arithmetic as moe_reference on the upcast values."""
    out = torch.zeros(x.shape, dtype=dtype)
    xf, wf = x.to(dtype), expert_weight.to(dtype)
    for e in range(w1.shape[0]):
        token, slot = torch.nonzero(expert_idx == e, as_tuple=True)
        if token.numel() == 0:
            continue
        y = F.gelu(xf[token] @ w1[e].to(dtype)) @ w2[e].to(dtype)
        out.index_add_(0, token, y * wf[token, slot, None])
    return out


def moe_assigned_reference(x, token_of_copy, expert_of_copy, weight_of_copy, w1, w2) -> torch.Tensor:
    """The layer on a flat assignment list, expert by expert: copy c sends token token_of_copy[c] to
    expert expert_of_copy[c] with weight weight_of_copy[c]; tokens without copies stay 0 (the check
    the reference's tests use for moe_forward_assigned: tests/test_token_rounding.py:90-97)."""
    out = torch.zeros(x.shape[0], x.shape[1], dtype=x.dtype)
    for e in range(w1.shape[0]):
        mask = expert_of_copy == e
        if mask.any():
            y = F.gelu(x[token_of_copy[mask]] @ w1[e]) @ w2[e]
            out.index_add_(0, token_of_copy[mask], y * weight_of_copy[mask, None].to(x.dtype))
    return out
