"""Block-sparse matmuls of the MoE layer: the reference's sparsebench/spmm.py surface."""

from __future__ import annotations

import torch

from sparsebench_b200 import _C
from sparsebench_b200.routing import DeviceTopology
from sparsebench_b200.topology import Topology


def dsd(blocks: torch.Tensor, w2_cat: torch.Tensor, topo: Topology | DeviceTopology, version: int = 1,
        skip_padding_rows: bool = False, layout_from_routing: bool = False) -> torch.Tensor:
    """out = H @ w2_cat with H block-sparse in topo's layout (reference: sparsebench/spmm.py:9-25).

    blocks [nnz, bs, bs] bf16, w2_cat [E*F, D] bf16 -> [num_row_blocks*bs, D] bf16. With a
    DeviceTopology everything is worst-case sized and nothing syncs. Rows of row blocks without
    blocks (past the real end) come out as zeros for versions 1-3 and are left unwritten from
    version 4 on: nothing downstream reads them.

    skip_padding_rows (not in the reference; the layer passes True): padding rows sit at the end of
    each row block in topo's layout, and a group of 32 rows that is all padding is then neither read
    from `blocks` nor written to the output, so those output rows are undefined instead of 0.

    layout_from_routing (not in the reference; the layer passes True): promises that topo is what
    route_device made (all row blocks of an expert share one list of column blocks), which lets layouts
    with several row blocks per expert run two row blocks per tile on pairs of thread blocks. Same result.
    """
    bs = topo.block_size
    if blocks.dim() != 3 or tuple(blocks.shape[1:]) != (bs, bs):
        raise ValueError(f"blocks must be [nnz, {bs}, {bs}] for this topology, got {tuple(blocks.shape)}")
    return _C.dsd_cuda(blocks, w2_cat, topo.row_offsets, topo.col_indices, version,
                       topo.row_token if skip_padding_rows else None,
                       topo.padded_offsets if layout_from_routing else None)


def sdd(x: torch.Tensor, w1: torch.Tensor, topo: Topology | DeviceTopology, gelu: bool = True,
        skip_padding_rows: bool = False, layout_from_routing: bool = False) -> torch.Tensor:
    """H = (gelu)(x[row_token] @ w1[expert]) on topo's blocks (reference: sparsebench/spmm.py:28-43).

    x [T, D] bf16, w1 [E, D, F] bf16 -> blocks [nnz, 128, 128] bf16 in topo's BSR order, ready for
    dsd(). Token rows are gathered inside the kernel's loads; padding rows come out exactly zero.
    With a DeviceTopology nothing syncs and blocks of dead row blocks are left unwritten. Needs
    block size 128, D % 64 == 0 and F % 256 == 0.

    skip_padding_rows (not in the reference; the layer passes True): a group of 32 rows that is all
    padding is not stored, so those rows of the blocks are undefined instead of 0; only a dsd() with
    the same flag may consume such blocks.

    layout_from_routing (not in the reference; the layer passes True): as for dsd().
    """
    if topo.block_size != 128:
        raise ValueError(f"sdd needs block size 128, got {topo.block_size}")
    return _C.sdd_cuda(x, w1, topo.row_token, topo.row_block_expert, topo.row_offsets, topo.col_indices.numel(), gelu,
                       skip_padding_rows, topo.padded_offsets if layout_from_routing else None)


def combine(y: torch.Tensor, expert_weight: torch.Tensor, topo: Topology | DeviceTopology) -> torch.Tensor:
    """[P, D] expert outputs -> [T, D]: each token's k rows, gate-weighted and summed in fp32
    (reference: sparsebench/moe.py:51-55), as one bandwidth-bound kernel."""
    return _C.combine_cuda(y, topo.copy_row, expert_weight)
