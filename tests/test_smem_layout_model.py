"""Host-side model of the shared-memory operand layouts the matmul kernels rely on, with a planted-bug control.

No memory checker is available for these kernels, and a wrong swizzle or descriptor stride shows up on the GPU only
as "numbers are off". This test restates, in numpy, (1) where the producers put every element of a stage (the SDD
gather warps' cp.async destinations, the 128-byte-swizzled TMA boxes of the weight tiles) and (2) where a tcgen05
shared-memory descriptor with the kernel's parameters (start address, leading / stride byte offsets, 128-byte
swizzle) makes the tensor core look for element (row, k) of A (K-major) and (k, n) of B (MN-major), and checks that
the two agree for every element and every 16-wide K slice. The control plants the classic mistakes (a swizzle on the
wrong row bits, a stride off by one group) and requires the model to catch them.
The constants mirror sparsebench_b200/csrc/bsr_gemm.cuh: stage A = 128 rows x 128 B, B = slabs of 64 k-rows x 128 B
(64 n each), K-major A with SBO 1024, MN-major B with SBO 1024 and LBO = one slab, advance of 32 B (A) and 2048 B
(B) per 16-wide K slice.
"""

import numpy as np
import pytest

TILE_M, TILE_K, SLAB_N, UMMA_K = 128, 64, 64, 16


def swizzle128(addr: np.ndarray | int):
    """The 128-byte swizzle on a byte address: 16-byte chunk index (bits 4-6) XOR row-in-group (bits 7-9)."""
    return addr ^ (((addr >> 7) & 7) << 4)


def gather_stage(x_rows: np.ndarray, row_bits: int = 7) -> np.ndarray:
    """What the SDD gather warps leave in an A stage: chunk c (8 bf16 = 16 B) of row r at r*128 + ((c ^ (r & 7)) << 4).
    x_rows: [128, 64] element ids. Returns the stage as 8192 2-byte cells."""
    stage = np.full(TILE_M * TILE_K, -1, dtype=np.int64)
    for r in range(TILE_M):
        for c in range(8):
            byte = r * 128 + ((c ^ (r & row_bits)) << 4)
            stage[byte // 2: byte // 2 + 8] = x_rows[r, c * 8:(c + 1) * 8]
    return stage


def tma_box(tile: np.ndarray) -> np.ndarray:
    """A 128-byte-swizzled TMA box of [rows, 64] 2-byte elements: element (r, e) at swizzle128(r*128 + 2e)."""
    rows = tile.shape[0]
    out = np.full(rows * 64, -1, dtype=np.int64)
    r, e = np.meshgrid(np.arange(rows), np.arange(64), indexing="ij")
    out[swizzle128(r * 128 + 2 * e) // 2] = tile
    return out


def read_a_kmajor(stage: np.ndarray, start: int, sbo: int = 1024) -> np.ndarray:
    """[128 rows, 16 k] as a K-major, 128B-swizzled descriptor at byte `start` addresses them."""
    r, k = np.meshgrid(np.arange(TILE_M), np.arange(UMMA_K), indexing="ij")
    addr = start + (r // 8) * sbo + (r % 8) * 128 + 2 * k
    return stage[swizzle128(addr) // 2]


def read_b_mnmajor(stage: np.ndarray, start: int, n_cols: int, lbo: int, sbo: int = 1024) -> np.ndarray:
    """[16 k, n_cols] as an MN-major, 128B-swizzled descriptor addresses them: 64 n per 128-byte row of a slab, groups
    of 8 k-rows `sbo` apart, slabs `lbo` apart."""
    k, n = np.meshgrid(np.arange(UMMA_K), np.arange(n_cols), indexing="ij")
    addr = start + (n // SLAB_N) * lbo + (k // 8) * sbo + (k % 8) * 128 + 2 * (n % SLAB_N)
    return stage[swizzle128(addr) // 2]


def test_gathered_a_rows_are_where_the_descriptor_reads_them() -> None:
    x_rows = np.arange(TILE_M * TILE_K).reshape(TILE_M, TILE_K)
    stage = gather_stage(x_rows)
    assert (stage >= 0).all(), "every cell of the stage is written exactly once"
    for kk in range(TILE_K // UMMA_K):
        assert np.array_equal(read_a_kmajor(stage, kk * 32), x_rows[:, kk * 16:(kk + 1) * 16]), kk


def test_tma_loaded_h_block_matches_the_gather_layout() -> None:
    # DSD stages A by TMA (box {64 k, 128 rows}); it must land exactly where the gather warps would put it.
    x_rows = np.arange(TILE_M * TILE_K).reshape(TILE_M, TILE_K)
    assert np.array_equal(tma_box(x_rows), gather_stage(x_rows))


@pytest.mark.parametrize("slabs", [2, 4])  # 4: one-CTA tile (N = 256); 2: a CTA's half in the pair kernel
def test_weight_slabs_are_where_the_mn_major_descriptor_reads_them(slabs: int) -> None:
    n_cols = slabs * SLAB_N
    w = np.arange(TILE_K * n_cols).reshape(TILE_K, n_cols)  # [k, n], n contiguous as in w1 / w2
    slab_cells = TILE_K * 64
    stage = np.concatenate([tma_box(w[:, j * 64:(j + 1) * 64]) for j in range(slabs)])  # one box {64 n, 64 k} per slab
    for kk in range(TILE_K // UMMA_K):
        got = read_b_mnmajor(stage, kk * 2048, n_cols, lbo=slab_cells * 2)
        assert np.array_equal(got, w[kk * 16:(kk + 1) * 16]), kk


def agrees(read, expected: np.ndarray) -> bool:
    try:
        return bool(np.array_equal(read(), expected))
    except IndexError:  # the descriptor walked out of the stage: also a caught bug
        return False


def test_the_model_catches_planted_layout_bugs() -> None:
    x_rows = np.arange(TILE_M * TILE_K).reshape(TILE_M, TILE_K)
    good = gather_stage(x_rows)
    assert agrees(lambda: read_a_kmajor(good, 0), x_rows[:, :16])
    # 1. swizzle on two row bits instead of three (writer and reader disagree for rows 4-7 of every group)
    assert not agrees(lambda: read_a_kmajor(gather_stage(x_rows, row_bits=3), 0), x_rows[:, :16])
    # 2. stride between 8-row groups off by one row
    assert not agrees(lambda: read_a_kmajor(good, 0, sbo=1024 + 128), x_rows[:, :16])
    # 3. K-slice advance of 16 B instead of 32 B
    assert not agrees(lambda: read_a_kmajor(good, 16), x_rows[:, 16:32])
    # 4. B: slab distance confused with the group distance
    w = np.arange(TILE_K * 256).reshape(TILE_K, 256)
    stage = np.concatenate([tma_box(w[:, j * 64:(j + 1) * 64]) for j in range(4)])
    assert agrees(lambda: read_b_mnmajor(stage, 0, 256, lbo=TILE_K * 128), w[:16])
    assert not agrees(lambda: read_b_mnmajor(stage, 0, 256, lbo=1024), w[:16])
