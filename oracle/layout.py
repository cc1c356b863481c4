"""Integer side of the oracle: routing decisions -> block-sparse layout, in numpy.

TEST INFRASTRUCTURE (see oracle/__init__.py). Restates
  * topology.build_topology            (reference: sparsebench/topology.py:53-118)
  * the worst-case device buffers of   build_topology_cuda (reference: csrc/routing.cu:197-281)
  * bsr_to_dense / dense_to_bsr        (reference: sparsebench/topology.py:127-145)

A "copy" is one (token, choice) pair, c = t*k + j. Copies are ordered by expert, ascending c inside
an expert (a stable sort), and each expert's group is padded to a multiple of block_size.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Layout:
    """All arrays int32. Trimmed to the real sizes (P rows) unless built by device_layout()."""

    block_size: int
    num_experts: int
    ffn_blocks: int
    tokens_per_expert: np.ndarray  # [E]
    padded_offsets: np.ndarray  # [E+1]
    row_token: np.ndarray  # [P]   -1 = padding
    copy_row: np.ndarray  # [T*k]
    row_block_expert: np.ndarray  # [P/bs]
    row_offsets: np.ndarray  # [P/bs + 1]
    col_indices: np.ndarray  # [P/bs * ffn_blocks]
    error: int = 0  # device_layout() only: 1 if an expert id was out of range

    @property
    def num_rows(self) -> int:
        return int(self.row_token.shape[0])

    @property
    def num_row_blocks(self) -> int:
        return int(self.row_block_expert.shape[0])

    @property
    def nnz_blocks(self) -> int:
        return int(self.col_indices.shape[0])

    FIELDS = ("tokens_per_expert", "padded_offsets", "row_token", "copy_row", "row_block_expert", "row_offsets",
              "col_indices")


def _sorted_layout(flat: np.ndarray, valid: np.ndarray, k: int, num_experts: int, ffn_blocks: int, block_size: int):
    """Shared core. `flat` int64 [n]; copies with valid == False are skipped."""
    n = flat.shape[0]
    kept = np.nonzero(valid)[0]  # ascending copy index
    experts = flat[kept]
    counts = np.bincount(experts, minlength=num_experts).astype(np.int64)
    padded = (counts + block_size - 1) // block_size * block_size
    offsets = np.zeros(num_experts + 1, dtype=np.int64)
    np.cumsum(padded, out=offsets[1:])
    num_rows = int(offsets[-1])

    # Stable sort by expert: ties keep ascending copy index (reference: topology.py:83-89).
    order = np.argsort(experts, kind="stable")
    sorted_expert = experts[order]
    first_of_expert = np.cumsum(counts) - counts
    rank = np.arange(kept.shape[0], dtype=np.int64) - first_of_expert[sorted_expert]
    dest = offsets[sorted_expert] + rank

    copy_row = np.full(n, -1, dtype=np.int64)
    copy_row[kept[order]] = dest
    row_token = np.full(num_rows, -1, dtype=np.int64)
    row_token[dest] = kept[order] // k

    row_block_expert = np.repeat(np.arange(num_experts, dtype=np.int64), padded // block_size)
    row_offsets = np.arange(row_block_expert.shape[0] + 1, dtype=np.int64) * ffn_blocks
    col_indices = (row_block_expert[:, None] * ffn_blocks + np.arange(ffn_blocks, dtype=np.int64)[None, :]).reshape(-1)
    return counts, offsets, row_token, copy_row, row_block_expert, row_offsets, col_indices


def _validate(expert_idx: np.ndarray, num_experts: int, ffn_dim: int, block_size: int) -> None:
    if expert_idx.ndim != 2 or expert_idx.shape[0] == 0 or expert_idx.shape[1] == 0:
        raise ValueError(f"expert_idx must be [T, k] with T, k > 0, got {expert_idx.shape}")
    if expert_idx.dtype not in (np.int32, np.int64):
        raise TypeError(f"expert_idx must be int32 or int64, got {expert_idx.dtype}")
    if num_experts <= 0 or block_size <= 0:
        raise ValueError("num_experts and block_size must be positive")
    if ffn_dim <= 0 or ffn_dim % block_size != 0:
        raise ValueError(f"ffn_dim ({ffn_dim}) must be a positive multiple of block_size ({block_size})")


def build_topology(expert_idx, num_experts: int, ffn_dim: int, block_size: int) -> Layout:
    """expert_idx [T, k] (numpy int32/int64 or a CPU torch tensor) -> trimmed Layout.
    Raises like the reference for bad shapes, dtypes, ranges and int32 overflow
    (sparsebench/topology.py:57-81)."""
    idx = np.asarray(expert_idx.cpu().numpy() if hasattr(expert_idx, "cpu") else expert_idx)
    _validate(idx, num_experts, ffn_dim, block_size)
    lo, hi = int(idx.min()), int(idx.max())
    if lo < 0 or hi >= num_experts:
        raise ValueError(f"expert ids must be in [0, {num_experts}), got range [{lo}, {hi}]")
    k = idx.shape[1]
    flat = idx.reshape(-1).astype(np.int64)
    ffn_blocks = ffn_dim // block_size
    parts = _sorted_layout(flat, np.ones(flat.shape[0], dtype=bool), k, num_experts, ffn_blocks, block_size)
    if int(parts[1][-1]) * ffn_dim >= 2**31:
        raise ValueError("problem too large for int32 indexing")
    return Layout(block_size, num_experts, ffn_blocks, *(p.astype(np.int32) for p in parts))


def worst_case_sizes(n_copies: int, num_experts: int, ffn_dim: int, block_size: int) -> tuple[int, int, int]:
    """(max_row_blocks, max_rows, ffn_blocks) as the device path sizes its buffers
    (reference: csrc/routing.cu:213-217)."""
    max_row_blocks = (n_copies + num_experts * (block_size - 1)) // block_size
    return max_row_blocks, max_row_blocks * block_size, ffn_dim // block_size


def device_layout(expert_idx, num_experts: int, ffn_dim: int, block_size: int) -> Layout:
    """What the device routing must leave in its worst-case sized buffers, tails included
    (reference: csrc/routing.cu:44-51,125-129,157-159,174-192,249):
      copies with an id outside [0, E) are skipped, get copy_row = -1 and set error = 1;
      row_token = -1 for padding rows and every row past the real end;
      row_block_expert = -1 and col_indices = -1 past the real end;
      row_offsets[i] = min(i, real_row_blocks) * ffn_blocks.
    """
    idx = np.asarray(expert_idx.cpu().numpy() if hasattr(expert_idx, "cpu") else expert_idx)
    _validate(idx, num_experts, ffn_dim, block_size)
    k = idx.shape[1]
    flat = idx.reshape(-1).astype(np.int64)
    valid = (flat >= 0) & (flat < num_experts)
    ffn_blocks = ffn_dim // block_size
    counts, offsets, row_token, copy_row, rbe, row_offsets, col_indices = _sorted_layout(
        np.where(valid, flat, 0), valid, k, num_experts, ffn_blocks, block_size)
    max_rb, max_rows, _ = worst_case_sizes(flat.shape[0], num_experts, ffn_dim, block_size)
    real_rb = rbe.shape[0]

    def pad(a: np.ndarray, size: int) -> np.ndarray:
        out = np.full(size, -1, dtype=np.int64)
        out[: a.shape[0]] = a
        return out

    full_offsets = np.minimum(np.arange(max_rb + 1, dtype=np.int64), real_rb) * ffn_blocks
    return Layout(
        block_size, num_experts, ffn_blocks,
        counts.astype(np.int32), offsets.astype(np.int32), pad(row_token, max_rows).astype(np.int32),
        copy_row.astype(np.int32), pad(rbe, max_rb).astype(np.int32), full_offsets.astype(np.int32),
        pad(col_indices, max_rb * ffn_blocks).astype(np.int32), error=int(not valid.all()),
    )


def _row_block_of_nnz(layout: Layout) -> np.ndarray:
    per_row = np.diff(layout.row_offsets.astype(np.int64))
    return np.repeat(np.arange(layout.num_row_blocks, dtype=np.int64), per_row)


def bsr_to_dense(blocks: np.ndarray, layout: Layout) -> np.ndarray:
    """[nnz, bs, bs] -> dense [P, E*F], zeros outside the layout (reference: topology.py:127-135)."""
    bs = layout.block_size
    if blocks.shape != (layout.nnz_blocks, bs, bs):
        raise ValueError(f"expected blocks of shape {(layout.nnz_blocks, bs, bs)}, got {blocks.shape}")
    col_blocks = layout.num_experts * layout.ffn_blocks
    grid = np.zeros((layout.num_row_blocks, col_blocks, bs, bs), dtype=blocks.dtype)
    grid[_row_block_of_nnz(layout), layout.col_indices.astype(np.int64)] = blocks
    return grid.transpose(0, 2, 1, 3).reshape(layout.num_rows, col_blocks * bs)


def dense_to_bsr(dense: np.ndarray, layout: Layout) -> np.ndarray:
    """Dense [P, E*F] -> [nnz, bs, bs]; values outside the layout are dropped
    (reference: topology.py:138-145)."""
    bs = layout.block_size
    col_blocks = layout.num_experts * layout.ffn_blocks
    if dense.shape != (layout.num_rows, col_blocks * bs):
        raise ValueError(f"expected dense of shape {(layout.num_rows, col_blocks * bs)}, got {dense.shape}")
    grid = dense.reshape(layout.num_row_blocks, bs, col_blocks, bs).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(grid[_row_block_of_nnz(layout), layout.col_indices.astype(np.int64)])
