"""The layout hand-off type of the block-sparse MoE path.

`Topology` has the fields, names and dtypes of the reference's dataclass
(sparsebench/topology.py:25-51): P padded rows split into row blocks that each belong to one expert,
stored as BSR (row_offsets / col_indices). Only the data type lives here; the CPU construction of
a layout is test infrastructure and is not part of this package.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Topology:
    block_size: int  # rows (and columns) of one block of H
    num_experts: int
    ffn_blocks: int  # how many blocks one expert's F columns make: F // block_size

    # Where the copies went. All int32.
    tokens_per_expert: torch.Tensor  # [E] copies routed to each expert, before padding
    padded_offsets: torch.Tensor  # [E+1] row at which each expert's group starts; the last entry is P
    row_token: torch.Tensor  # [P] which token a row holds; -1 marks a row that only pads its group
    copy_row: torch.Tensor  # [T*k] the row that copy j of token t (index t*k + j) landed in

    # H as a block-sparse matrix: row block rb owns blocks row_offsets[rb] .. row_offsets[rb+1], the block at
    # position p sits in block column col_indices[p] (its expert's columns).
    row_block_expert: torch.Tensor  # [P / block_size] the expert a row block belongs to
    row_offsets: torch.Tensor  # [P / block_size + 1]
    col_indices: torch.Tensor  # [nnz_blocks]

    @property
    def num_rows(self) -> int:
        return self.row_token.numel()

    @property
    def num_row_blocks(self) -> int:
        return self.row_block_expert.numel()

    @property
    def nnz_blocks(self) -> int:
        return self.col_indices.numel()
