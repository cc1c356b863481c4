"""The operator surface of the reference's one extension module, `sparsebench._C`
(csrc/bindings.cpp:5-16, csrc/ops.hpp:11-36), on top of libsparsebench_b200's C ABI.

Same function names, positional order, keyword names, return shapes and error behaviour: argument
errors raise RuntimeError whose text contains what the reference's TORCH_CHECK messages contain;
data errors (an expert id out of range) never raise. Each call checks its arguments on the host,
allocates its outputs from torch's caching allocator on the input's device (so it can be captured
in a CUDA graph), and enqueues kernels on torch's current stream. Nothing here synchronises,
copies to the host or reads a size back from the GPU.
"""

from __future__ import annotations

import ctypes

import torch

from sparsebench_b200 import _lib

BLOCK = 128  # the block size the two matmuls are built for

_dev_status: dict[int, torch.Tensor] = {}


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise RuntimeError(message)


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None or t.numel() == 0 else t.data_ptr())


def device_status(device: torch.device) -> torch.Tensor:
    """int32[1] on `device` that the matmul kernels OR a non-zero code into if one of their bounded
    device-side waits ever expires. Allocated zeroed on first use; reading it syncs."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _dev_status:
        _dev_status[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return _dev_status[index]


def arch_probe(n: int) -> torch.Tensor:
    """int32[n] filled with __CUDA_ARCH__ of the device code that ran (1000 on B200).
    Reference: csrc/smoke.cu:23-38."""
    lib = _lib.load()
    _check(n > 0, f"arch_probe: n must be positive, got {n}")
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    _lib.check(lib.sb_arch_probe(_ptr(out), n, _stream()))
    return out


def build_topology_cuda(expert_idx: torch.Tensor, num_experts: int, ffn_dim: int, block_size: int) -> list[torch.Tensor]:
    """Routing -> block-sparse layout on the GPU, no host sync. Reference: csrc/routing.cu:197-281.

    Returns [tokens_per_expert[E], padded_offsets[E+1], row_token[max_rows], copy_row[T*k],
    row_block_expert[max_rb], row_offsets[max_rb+1], col_indices[max_rb*ffn_blocks], error[1]],
    all int32 on expert_idx's device and sized for the worst case.
    """
    lib = _lib.load()
    _check(isinstance(expert_idx, torch.Tensor) and expert_idx.is_cuda, "expert_idx must be a CUDA tensor")
    _check(expert_idx.dim() == 2 and expert_idx.shape[0] > 0 and expert_idx.shape[1] > 0,
           f"expert_idx must be [T, k] with T, k > 0, got {tuple(expert_idx.shape)}")
    _check(expert_idx.dtype in (torch.int32, torch.int64),
           f"expert_idx must be int32 or int64, got {expert_idx.dtype}")
    _check(expert_idx.is_contiguous(), "expert_idx must be contiguous")

    n, k = expert_idx.numel(), expert_idx.shape[1]
    max_rb, max_rows, ffn_blocks = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _lib.check(lib.sb_route_sizes(n, num_experts, ffn_dim, block_size, ctypes.byref(max_rb), ctypes.byref(max_rows),
                                  ctypes.byref(ffn_blocks)))
    max_rb, max_rows, ffn_blocks = max_rb.value, max_rows.value, ffn_blocks.value
    work_ints = (lib.sb_route_workspace_bytes(n, num_experts) + 3) // 4

    with torch.cuda.device(expert_idx.device):
        # One allocation, carved into the eight outputs (+ scratch): fewer allocator calls per layer.
        sizes = [num_experts, num_experts + 1, max_rows, n, max_rb, max_rb + 1, max_rb * ffn_blocks, 1, work_ints]
        buf = torch.empty(sum(sizes), dtype=torch.int32, device=expert_idx.device)
        parts = list(torch.split(buf, sizes))
        work = parts.pop()
        _lib.check(lib.sb_route(_ptr(expert_idx), int(expert_idx.dtype == torch.int64), n, k, num_experts, ffn_blocks,
                                block_size, max_rb, *(_ptr(t) for t in parts), _ptr(work), _stream()))
    return parts


def _check_index(t: torch.Tensor, name: str) -> None:
    _check(t.is_cuda and t.dtype == torch.int32 and t.dim() == 1 and t.is_contiguous(),
           f"{name} must be a contiguous 1-D int32 CUDA tensor")


def sdd_cuda(x: torch.Tensor, w1: torch.Tensor, row_token: torch.Tensor, row_block_expert: torch.Tensor,
             row_offsets: torch.Tensor, num_nnz: int, apply_gelu: bool) -> torch.Tensor:
    """Blocks [num_nnz, 128, 128] = (gelu)(x[row_token] @ w1[expert]) on the layout's blocks.
    Reference: csrc/sdd.cu:123-170. Blocks of dead row blocks are left unwritten."""
    lib = _lib.load()
    _check(x.is_cuda and w1.is_cuda and x.device == w1.device, "x and w1 must be on the same GPU (CUDA tensors)")
    _check(x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16, "x and w1 must be bfloat16")
    _check(x.is_contiguous() and w1.is_contiguous(), "x and w1 must be contiguous")
    _check(x.dim() == 2 and w1.dim() == 3 and w1.shape[1] == x.shape[1],
           f"x must be [T, D] and w1 [E, D, F], got {tuple(x.shape)} and {tuple(w1.shape)}")
    _check_index(row_token, "row_token")
    _check_index(row_block_expert, "row_block_expert")
    _check_index(row_offsets, "row_offsets")
    d_model, ffn_dim = x.shape[1], w1.shape[2]
    num_row_blocks = row_offsets.numel() - 1
    _check(d_model > 0 and d_model % 64 == 0, f"sdd needs D ({d_model}) to be a multiple of 64")
    _check(ffn_dim > 0 and ffn_dim % 256 == 0, f"sdd needs F ({ffn_dim}) to be a multiple of 256")
    _check(row_token.numel() == num_row_blocks * BLOCK,
           f"sdd needs block size 128: row_token has {row_token.numel()} rows for {num_row_blocks} row blocks")
    _check(row_block_expert.numel() == num_row_blocks, "row_block_expert must have one entry per row block")
    _check(num_nnz == num_row_blocks * (ffn_dim // BLOCK),
           f"expected {num_row_blocks * (ffn_dim // BLOCK)} blocks (row blocks x F/128), got {num_nnz}")

    with torch.cuda.device(x.device):
        out = torch.empty((num_nnz, BLOCK, BLOCK), dtype=torch.bfloat16, device=x.device)
        if num_row_blocks > 0:
            _lib.check(lib.sb_sdd(_ptr(x), _ptr(w1), _ptr(row_token), _ptr(row_block_expert), _ptr(row_offsets),
                                  _ptr(out), x.shape[0], d_model, ffn_dim, w1.shape[0], num_row_blocks,
                                  int(bool(apply_gelu)), _ptr(device_status(x.device)), _stream()))
    return out


_DSD_VERSIONS = {1, 2, 21, 3, 31, 4, 41, 5}
_DSD_ZERO_DEAD_ROWS = {1, 2, 21, 3, 31}


def dsd_cuda(blocks: torch.Tensor, w: torch.Tensor, row_offsets: torch.Tensor, col_indices: torch.Tensor,
             version: int) -> torch.Tensor:
    """out [num_row_blocks*bs, D] = BSR(blocks, row_offsets, col_indices) @ w.
    Reference: csrc/dsd.cpp:27-80. `version` keeps the reference's meaning for what is observable:
    versions 1, 2, 21, 3, 31 zero the rows of row blocks without blocks, 4, 41 and 5 leave them
    unwritten, 5 insists on block size 128 and D % 256 == 0; one tcgen05 kernel serves them all."""
    lib = _lib.load()
    _check(blocks.is_cuda and w.is_cuda, "blocks and w must be CUDA tensors")
    _check(blocks.device == w.device and row_offsets.device == w.device and col_indices.device == w.device,
           "all inputs must be on the same GPU")
    _check(blocks.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "blocks and w must be bfloat16")
    _check(blocks.is_contiguous() and w.is_contiguous(), "blocks and w must be contiguous")
    _check(blocks.dim() == 3 and blocks.shape[1] == blocks.shape[2],
           f"blocks must be [nnz, bs, bs], got {tuple(blocks.shape)}")
    _check(w.dim() == 2, f"w must be [E*F, D], got {tuple(w.shape)}")
    _check_index(row_offsets, "row_offsets")
    _check_index(col_indices, "col_indices")
    bs, d_model = blocks.shape[1], w.shape[1]
    num_row_blocks = row_offsets.numel() - 1
    _check(bs in (64, 128), f"block size must be 64 or 128, got {bs}")
    _check(d_model > 0 and d_model % 128 == 0, f"D ({d_model}) must be a positive multiple of 128")
    _check(w.shape[0] % bs == 0, f"w rows ({w.shape[0]}) must be a multiple of the block size ({bs})")
    _check(num_row_blocks >= 0, "row_offsets must have at least one entry")
    _check(blocks.shape[0] == col_indices.numel(),
           f"blocks has {blocks.shape[0]} blocks but col_indices has {col_indices.numel()}")
    _check(version in _DSD_VERSIONS, f"unknown dsd version {version}")
    if version == 5:
        _check(bs == 128 and d_model % 256 == 0,
               f"dsd v5 needs block size 128 and D a multiple of 256, got block size {bs}, D {d_model}")

    with torch.cuda.device(w.device):
        out = torch.empty((num_row_blocks * bs, d_model), dtype=torch.bfloat16, device=w.device)
        if num_row_blocks > 0:
            _lib.check(lib.sb_dsd(_ptr(blocks), blocks.shape[0], _ptr(w), w.shape[0], d_model, _ptr(row_offsets),
                                  _ptr(col_indices), num_row_blocks, bs, int(version in _DSD_ZERO_DEAD_ROWS),
                                  _ptr(out), _ptr(device_status(w.device)), _stream()))
    return out


def combine_cuda(y: torch.Tensor, copy_row: torch.Tensor, expert_weight: torch.Tensor) -> torch.Tensor:
    """out[t] = bf16(sum_j float(y[copy_row[t*k+j]]) * float(expert_weight[t, j])): the gate-weighted
    combine the reference does with PyTorch ops (sparsebench/moe.py:51-55), as one kernel."""
    lib = _lib.load()
    _check(y.is_cuda and copy_row.is_cuda and expert_weight.is_cuda, "combine inputs must be CUDA tensors")
    _check(y.dtype == torch.bfloat16 and y.dim() == 2 and y.is_contiguous(), "y must be a contiguous [P, D] bfloat16 tensor")
    _check(expert_weight.dim() == 2 and expert_weight.is_contiguous(), "expert_weight must be a contiguous [T, k] tensor")
    _check(expert_weight.dtype in (torch.bfloat16, torch.float32), "expert_weight must be bfloat16 or float32")
    _check_index(copy_row, "copy_row")
    num_tokens, k = expert_weight.shape
    _check(copy_row.numel() == num_tokens * k, "copy_row must have T*k entries")
    _check(y.shape[1] % 8 == 0, f"D ({y.shape[1]}) must be a multiple of 8")
    with torch.cuda.device(y.device):
        out = torch.empty((num_tokens, y.shape[1]), dtype=torch.bfloat16, device=y.device)
        if num_tokens > 0:
            _lib.check(lib.sb_combine(_ptr(y), _ptr(copy_row), _ptr(expert_weight),
                                      int(expert_weight.dtype == torch.float32), _ptr(out), num_tokens, k,
                                      y.shape[1], _stream()))
    return out
