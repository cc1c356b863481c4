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
    block_size: int
    num_experts: int
    ffn_blocks: int  # F // block_size: column blocks per expert

    tokens_per_expert: torch.Tensor  # [E] int32, real copies per expert
    padded_offsets: torch.Tensor  # [E+1] int32, first padded row of each expert
    row_token: torch.Tensor  # [P] int32, source token of each row, -1 = padding
    copy_row: torch.Tensor  # [T*k] int32, padded row of copy (t, j) at t*k + j

    row_block_expert: torch.Tensor  # [P / block_size] int32
    row_offsets: torch.Tensor  # [P / block_size + 1] int32
    col_indices: torch.Tensor  # [nnz_blocks] int32

    @property
    def num_rows(self) -> int:
        return self.row_token.numel()

    @property
    def num_row_blocks(self) -> int:
        return self.row_block_expert.numel()

    @property
    def nnz_blocks(self) -> int:
        return self.col_indices.numel()
