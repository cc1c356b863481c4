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
             row_offsets: torch.Tensor, num_nnz: int, apply_gelu: bool,
             skip_padding_rows: bool = False, padded_offsets: torch.Tensor | None = None) -> torch.Tensor:
    """Blocks [num_nnz, 128, 128] = (gelu)(x[row_token] @ w1[expert]) on the layout's blocks.
    Reference: csrc/sdd.cu:123-170. Blocks of dead row blocks are left unwritten; with
    skip_padding_rows so are groups of 32 rows that are all padding (padding at the end of each row
    block, as routing lays it out) instead of coming out 0. padded_offsets (routing's [E + 1] array):
    lets layouts with several row blocks per expert run two row blocks per tile on pairs of thread blocks."""
    lib = _lib.load()
    _check(x.is_cuda and w1.is_cuda and x.device == w1.device, "x and w1 must be on the same GPU (CUDA tensors)")
    _check(x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16, "x and w1 must be bfloat16")
    _check(x.is_contiguous() and w1.is_contiguous(), "x and w1 must be contiguous")
    _check(x.dim() == 2 and w1.dim() == 3 and w1.shape[1] == x.shape[1],
           f"x must be [T, D] and w1 [E, D, F], got {tuple(x.shape)} and {tuple(w1.shape)}")
    _check_index(row_token, "row_token")
    _check_index(row_block_expert, "row_block_expert")
    _check_index(row_offsets, "row_offsets")
    if padded_offsets is not None:
        _check_index(padded_offsets, "padded_offsets")
        _check(padded_offsets.numel() == w1.shape[0] + 1, "padded_offsets must have E + 1 entries")
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
                                  int(bool(apply_gelu)), int(bool(skip_padding_rows)),
                                  _ptr(padded_offsets) if padded_offsets is not None else None,
                                  _ptr(device_status(x.device)), _stream()))
    return out


_DSD_VERSIONS = {1, 2, 21, 3, 31, 4, 41, 5}
_DSD_ZERO_DEAD_ROWS = {1, 2, 21, 3, 31}


def dsd_cuda(blocks: torch.Tensor, w: torch.Tensor, row_offsets: torch.Tensor, col_indices: torch.Tensor,
             version: int, row_token: torch.Tensor | None = None,
             padded_offsets: torch.Tensor | None = None) -> torch.Tensor:
    """out [num_row_blocks*bs, D] = BSR(blocks, row_offsets, col_indices) @ w.
    Reference: csrc/dsd.cpp:27-80. `version` keeps the reference's meaning for what is observable:
    versions 1, 2, 21, 3, 31 zero the rows of row blocks without blocks, 4, 41 and 5 leave them
    unwritten, 5 insists on block size 128 and D % 256 == 0; one tcgen05 kernel serves them all.
    With row_token (the layout's row -> token table, padding at the end of each row block), groups of
    32 rows that are all padding are neither read nor written. padded_offsets (routing's [E + 1] array,
    only for a layout routing made): lets layouts with several row blocks per expert run on pairs of
    thread blocks."""
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
    if padded_offsets is not None:
        _check_index(padded_offsets, "padded_offsets")
    if row_token is not None:
        _check_index(row_token, "row_token")
        _check(row_token.device == w.device and row_token.numel() == num_row_blocks * bs,
               f"row_token must hold {num_row_blocks * bs} rows on the same GPU")

    with torch.cuda.device(w.device):
        out = torch.empty((num_row_blocks * bs, d_model), dtype=torch.bfloat16, device=w.device)
        if num_row_blocks > 0:
            _lib.check(lib.sb_dsd(_ptr(blocks), blocks.shape[0], _ptr(w), w.shape[0], d_model, _ptr(row_offsets),
                                  _ptr(col_indices), num_row_blocks, bs, int(version in _DSD_ZERO_DEAD_ROWS),
                                  _ptr(row_token) if row_token is not None else None, _ptr(out),
                                  _ptr(padded_offsets) if padded_offsets is not None else None,
                                  padded_offsets.numel() - 1 if padded_offsets is not None else 0,
                                  _ptr(device_status(w.device)), _stream()))
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


# ---- router front end (torch.topk + softmax in the reference, sparsebench/reference.py:19-29) ----------

def router_topk_cuda(logits: torch.Tensor, k: int, index_dtype: torch.dtype = torch.int64) -> tuple[torch.Tensor, torch.Tensor]:
    """(expert_idx [T, k], expert_weight [T, k]): the k largest logits per token and a softmax over them."""
    lib = _lib.load()
    _check(logits.is_cuda and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous [T, E] CUDA tensor")
    _check(logits.dtype in (torch.bfloat16, torch.float32), "logits must be bfloat16 or float32")
    _check(index_dtype in (torch.int32, torch.int64), "index_dtype must be int32 or int64")
    num_tokens, num_experts = logits.shape
    _check(0 < k <= num_experts, f"need [T, E] logits with 0 < k <= E, got {tuple(logits.shape)} and k={k}")
    with torch.cuda.device(logits.device):
        idx = torch.empty((num_tokens, k), dtype=index_dtype, device=logits.device)
        weight = torch.empty((num_tokens, k), dtype=logits.dtype, device=logits.device)
        if num_tokens > 0:
            _lib.check(lib.sb_router_topk(_ptr(logits), int(logits.dtype == torch.float32), num_tokens, num_experts, k,
                                          _ptr(idx), int(index_dtype == torch.int64), _ptr(weight), _stream()))
    return idx, weight


def route_from_logits_cuda(logits: torch.Tensor, k: int, ffn_dim: int, block_size: int, one_launch: bool = False):
    """(expert_idx [T, k] int64, expert_weight [T, k], the eight arrays of build_topology_cuda) from router
    logits [T, E]: router_topk_cuda followed by build_topology_cuda (6 + 10 us at T=4096, E=64 on a B200), or with
    one_launch a single kernel where that form applies (k in {1, 2, 4, 8}, E <= 1024, T*k <= 32768; 36 us there:
    the top-k then runs on the few thread blocks of the routing cluster). Same results either way."""
    lib = _lib.load()
    _check(logits.is_cuda and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous [T, E] CUDA tensor")
    _check(logits.dtype in (torch.bfloat16, torch.float32), "logits must be bfloat16 or float32")
    num_tokens, num_experts = logits.shape
    _check(0 < k <= num_experts, f"need [T, E] logits with 0 < k <= E, got {tuple(logits.shape)} and k={k}")
    if not one_launch or num_tokens == 0 or not lib.sb_route_from_logits_fused(num_tokens, k, num_experts):
        idx, weight = router_topk_cuda(logits, k)
        return idx, weight, build_topology_cuda(idx, num_experts, ffn_dim, block_size)
    n = num_tokens * k
    max_rb, max_rows, ffn_blocks = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _lib.check(lib.sb_route_sizes(n, num_experts, ffn_dim, block_size, ctypes.byref(max_rb), ctypes.byref(max_rows),
                                  ctypes.byref(ffn_blocks)))
    max_rb, max_rows, ffn_blocks = max_rb.value, max_rows.value, ffn_blocks.value
    with torch.cuda.device(logits.device):
        idx = torch.empty((num_tokens, k), dtype=torch.int64, device=logits.device)
        weight = torch.empty((num_tokens, k), dtype=logits.dtype, device=logits.device)
        sizes = [num_experts, num_experts + 1, max_rows, n, max_rb, max_rb + 1, max_rb * ffn_blocks, 1]
        parts = list(torch.split(torch.empty(sum(sizes), dtype=torch.int32, device=logits.device), sizes))
        _lib.check(lib.sb_route_from_logits(_ptr(logits), int(logits.dtype == torch.float32), num_tokens, k, num_experts,
                                            ffn_blocks, block_size, max_rb, _ptr(idx), _ptr(weight),
                                            *(_ptr(t) for t in parts), _stream()))
    return idx, weight, parts


# ---- the layer on a flat assignment list (PyTorch ops in the reference, sparsebench/moe.py:59-91) ---

def remap_rows_cuda(row_copy: torch.Tensor, token_of_copy: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """row_token[r] = token_of_copy[row_copy[r]] where row_copy[r] >= 0 and the token lies in
    [0, num_tokens), else -1."""
    lib = _lib.load()
    _check_index(row_copy, "row_copy")
    _check(token_of_copy.is_cuda and token_of_copy.dim() == 1 and token_of_copy.is_contiguous() and
           token_of_copy.dtype in (torch.int32, torch.int64), "token_of_copy must be a contiguous 1-D int32/int64 CUDA tensor")
    with torch.cuda.device(row_copy.device):
        out = torch.empty_like(row_copy)
        if row_copy.numel() > 0:
            _lib.check(lib.sb_remap_rows(_ptr(row_copy), _ptr(token_of_copy), int(token_of_copy.dtype == torch.int64),
                                         _ptr(out), row_copy.numel(), token_of_copy.numel(), num_tokens, _stream()))
    return out


def combine_assigned_cuda(y: torch.Tensor, copy_row: torch.Tensor, token_of_copy: torch.Tensor,
                          weight_of_copy: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """out[t] = bf16(sum over the copies c of token t of float(y[copy_row[c]]) * float(weight_of_copy[c]))."""
    lib = _lib.load()
    _check(y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.is_contiguous(),
           "y must be a contiguous [P, D] bfloat16 CUDA tensor")
    _check_index(copy_row, "copy_row")
    n = copy_row.numel()
    _check(token_of_copy.numel() == n and weight_of_copy.numel() == n, "token_of_copy and weight_of_copy need one entry per copy")
    _check(token_of_copy.dtype in (torch.int32, torch.int64) and token_of_copy.is_contiguous(),
           "token_of_copy must be contiguous int32/int64")
    if weight_of_copy.dtype not in (torch.bfloat16, torch.float32):
        weight_of_copy = weight_of_copy.float()
    weight_of_copy = weight_of_copy.contiguous()
    _check(y.shape[1] % 4 == 0, f"D ({y.shape[1]}) must be a multiple of 4")
    with torch.cuda.device(y.device):
        acc = torch.empty((num_tokens, y.shape[1]), dtype=torch.float32, device=y.device)
        out = torch.empty((num_tokens, y.shape[1]), dtype=torch.bfloat16, device=y.device)
        _lib.check(lib.sb_combine_assigned(_ptr(y), _ptr(copy_row), _ptr(token_of_copy),
                                           int(token_of_copy.dtype == torch.int64), _ptr(weight_of_copy),
                                           int(weight_of_copy.dtype == torch.float32), _ptr(acc), _ptr(out), n,
                                           num_tokens, y.shape[1], _stream()))
    return out


def token_rounding_cuda(scores: torch.Tensor, k: int, tile: int):
    """(token_of_copy int32 [cap], expert_of_copy int32 [cap], weight_of_copy fp32 [cap], num_copies int32 [1]) with
    cap = T*k + E*(tile // 2): the reference's token_rounding (sparsebench/token_rounding.py:58-81) without its host
    sync. Entries past num_copies carry expert -1 (skipped by routing) and weight 0."""
    lib = _lib.load()
    _check(scores.is_cuda and scores.dim() == 2 and scores.is_contiguous() and scores.dtype == torch.float32,
           "scores must be a contiguous [T, E] float32 CUDA tensor")
    num_tokens, num_experts = scores.shape
    _check(num_tokens > 0 and 0 < k <= num_experts and tile > 0, f"need [T, E] scores with 0 < k <= E and tile > 0, got k={k}")
    cap = lib.sb_token_rounding_capacity(num_tokens, num_experts, k, tile)
    work = lib.sb_token_rounding_workspace_bytes(num_tokens, num_experts, k)
    with torch.cuda.device(scores.device):
        token = torch.empty(cap, dtype=torch.int32, device=scores.device)
        expert = torch.empty(cap, dtype=torch.int32, device=scores.device)
        weight = torch.empty(cap, dtype=torch.float32, device=scores.device)
        count = torch.empty(1, dtype=torch.int32, device=scores.device)
        scratch = torch.empty((work + 3) // 4, dtype=torch.int32, device=scores.device)
        _lib.check(lib.sb_token_rounding(_ptr(scores), num_tokens, num_experts, k, tile, _ptr(token), _ptr(expert),
                                         _ptr(weight), _ptr(count), _ptr(scratch), _stream()))
    return token, expert, weight, count


# ---- expert-parallel plumbing (no counterpart in the reference's extension) ----------------------

def sort_copies_cuda(expert_idx: torch.Tensor, num_experts: int) -> list[torch.Tensor]:
    """Stable sort of the T*k copies by expert, nothing else: sb_route at block size 1 without the BSR
    arrays. Returns [tokens_per_expert[E], offsets[E+1] (exclusive scan of the counts),
    sorted_token[T*k] (-1 past the kept copies), copy_pos[T*k] (-1 for a rejected id), error[1]]."""
    lib = _lib.load()
    _check(expert_idx.is_cuda and expert_idx.dim() == 2 and expert_idx.is_contiguous() and
           expert_idx.dtype in (torch.int32, torch.int64), "expert_idx must be a contiguous [T, k] int32/int64 CUDA tensor")
    n, k = expert_idx.numel(), expert_idx.shape[1]
    _check(n > 0, "expert_idx must be [T, k] with T, k > 0")
    max_rb = ctypes.c_int64()
    _lib.check(lib.sb_route_sizes(n, num_experts, 1, 1, ctypes.byref(max_rb), None, None))
    work_ints = (lib.sb_route_workspace_bytes(n, num_experts) + 3) // 4
    with torch.cuda.device(expert_idx.device):
        sizes = [num_experts, num_experts + 1, n, n, 1, work_ints]
        parts = list(torch.split(torch.empty(sum(sizes), dtype=torch.int32, device=expert_idx.device), sizes))
        work = parts.pop()
        counts, offsets, sorted_token, copy_pos, error = parts
        _lib.check(lib.sb_route(_ptr(expert_idx), int(expert_idx.dtype == torch.int64), n, k, num_experts, 1, 1,
                                max_rb.value, _ptr(counts), _ptr(offsets), _ptr(sorted_token), _ptr(copy_pos),
                                None, None, None, _ptr(error), _ptr(work), _stream()))
    return parts


def ep_plan(expert_offsets: torch.Tensor, sorted_token: torch.Tensor, copy_pos: torch.Tensor, num_ranks: int,
            experts_per_rank: int, capacity: int, status: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(send_index [N*C], return_row [n]) from a rank's block-size-1 sort by global expert."""
    lib = _lib.load()
    for t, name in ((expert_offsets, "expert_offsets"), (sorted_token, "sorted_token"), (copy_pos, "copy_pos"),
                    (status, "status")):
        _check_index(t, name)
    _check(expert_offsets.numel() == num_ranks * experts_per_rank + 1, "expert_offsets must have E + 1 entries")
    n = copy_pos.numel()
    with torch.cuda.device(copy_pos.device):
        send_index = torch.empty(num_ranks * capacity, dtype=torch.int32, device=copy_pos.device)
        return_row = torch.empty(n, dtype=torch.int32, device=copy_pos.device)
        _lib.check(lib.sb_ep_plan(_ptr(expert_offsets), _ptr(sorted_token), _ptr(copy_pos), n, num_ranks,
                                  experts_per_rank, capacity, _ptr(send_index), _ptr(return_row), _ptr(status),
                                  _stream()))
    return send_index, return_row


def ep_slot_experts(recv_counts: torch.Tensor, capacity: int) -> torch.Tensor:
    """recv_counts [N, E_local] int32 -> slot_expert [N*capacity] int32 (-1 for empty slots)."""
    lib = _lib.load()
    _check(recv_counts.is_cuda and recv_counts.dtype == torch.int32 and recv_counts.dim() == 2 and
           recv_counts.is_contiguous(), "recv_counts must be a contiguous [N, E_local] int32 CUDA tensor")
    num_ranks, experts_per_rank = recv_counts.shape
    with torch.cuda.device(recv_counts.device):
        out = torch.empty(num_ranks * capacity, dtype=torch.int32, device=recv_counts.device)
        _lib.check(lib.sb_ep_slot_experts(_ptr(recv_counts), num_ranks, experts_per_rank, capacity, _ptr(out), _stream()))
    return out


def gather_rows(src: torch.Tensor, index: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[j] = src[index[j]] where index[j] >= 0; other rows keep what they held."""
    lib = _lib.load()
    _check(src.is_cuda and src.dim() == 2 and src.is_contiguous(), "src must be a contiguous 2-D CUDA tensor")
    _check_index(index, "index")
    row_bytes = src.shape[1] * src.element_size()
    _check(row_bytes % 16 == 0, f"row size ({row_bytes} bytes) must be a multiple of 16")
    with torch.cuda.device(src.device):
        if out is None:
            out = torch.empty((index.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
        _check(out.is_contiguous() and out.shape == (index.numel(), src.shape[1]) and out.dtype == src.dtype,
               "out must be a contiguous [len(index), row] tensor of src's dtype")
        if index.numel() > 0:
            _lib.check(lib.sb_gather_rows(_ptr(src), _ptr(index), _ptr(out), index.numel(), row_bytes, _stream()))
    return out


def ep_push_rows(src: torch.Tensor, index: torch.Tensor, peer_base: torch.Tensor, my_rank: int, capacity: int) -> None:
    """Row src[index[j]] of every slot j = peer*capacity + i with index[j] >= 0 is stored into rank
    `peer`'s buffer (peer_base[peer], an int64 device array of mapped base addresses) at row
    my_rank*capacity + i."""
    lib = _lib.load()
    _check(src.is_cuda and src.dim() == 2 and src.is_contiguous(), "src must be a contiguous 2-D CUDA tensor")
    _check_index(index, "index")
    _check(peer_base.is_cuda and peer_base.dtype == torch.int64 and peer_base.is_contiguous(),
           "peer_base must be a contiguous int64 CUDA tensor of base addresses")
    num_ranks = peer_base.numel()
    _check(index.numel() == num_ranks * capacity, "index must have ranks * capacity entries")
    with torch.cuda.device(src.device):
        _lib.check(lib.sb_ep_push_rows(_ptr(src), _ptr(index), _ptr(peer_base), my_rank, num_ranks, capacity,
                                       src.shape[1] * src.element_size(), _stream()))


def ep_dsd_push(blocks: torch.Tensor, w: torch.Tensor, row_offsets: torch.Tensor, col_indices: torch.Tensor,
                row_slot: torch.Tensor, peer_base: torch.Tensor, my_rank: int, capacity: int) -> None:
    """DSD whose epilogue stores row r of the layout into rank (row_slot[r] // capacity)'s buffer
    (peer_base, an int64 device array of mapped base addresses) at row my_rank*capacity +
    row_slot[r] % capacity: dsd_cuda + ep_push_rows as one kernel. Block size 128."""
    lib = _lib.load()
    _check(blocks.is_cuda and w.is_cuda and blocks.device == w.device, "blocks and w must be on the same GPU")
    _check(blocks.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "blocks and w must be bfloat16")
    _check(blocks.is_contiguous() and w.is_contiguous(), "blocks and w must be contiguous")
    _check(blocks.dim() == 3 and tuple(blocks.shape[1:]) == (BLOCK, BLOCK), f"blocks must be [nnz, 128, 128], got {tuple(blocks.shape)}")
    _check(w.dim() == 2 and w.shape[1] % 128 == 0, f"w must be [E*F, D] with D a multiple of 128, got {tuple(w.shape)}")
    for t, name in ((row_offsets, "row_offsets"), (col_indices, "col_indices"), (row_slot, "row_slot")):
        _check_index(t, name)
    num_row_blocks = row_offsets.numel() - 1
    _check(row_slot.numel() == num_row_blocks * BLOCK, f"row_slot must hold {num_row_blocks * BLOCK} rows")
    _check(blocks.shape[0] == col_indices.numel(), "blocks and col_indices disagree")
    _check(peer_base.is_cuda and peer_base.dtype == torch.int64 and peer_base.is_contiguous(),
           "peer_base must be a contiguous int64 CUDA tensor of base addresses")
    with torch.cuda.device(w.device):
        if num_row_blocks > 0:
            _lib.check(lib.sb_ep_dsd_push(_ptr(blocks), blocks.shape[0], _ptr(w), w.shape[0], w.shape[1],
                                          _ptr(row_offsets), _ptr(col_indices), num_row_blocks, _ptr(row_slot),
                                          _ptr(peer_base), my_rank, peer_base.numel(), capacity,
                                          _ptr(device_status(w.device)), _stream()))


def ep_push_counts(counts: torch.Tensor, peer_counts: torch.Tensor, my_rank: int, experts_per_rank: int) -> None:
    """counts[d*E_local + e] -> rank d's table (peer_counts[d]) at [my_rank*E_local + e]."""
    lib = _lib.load()
    _check_index(counts, "counts")
    num_ranks = peer_counts.numel()
    _check(counts.numel() == num_ranks * experts_per_rank, "counts must have ranks * experts_per_rank entries")
    with torch.cuda.device(counts.device):
        _lib.check(lib.sb_ep_push_counts(_ptr(counts), _ptr(peer_counts), my_rank, num_ranks, experts_per_rank, _stream()))


def ep_barrier(peer_pads: torch.Tensor, my_pad: torch.Tensor, epoch: torch.Tensor, my_rank: int,
               status: torch.Tensor) -> None:
    """Device-side barrier of all ranks over peer memory (bounded wait; see sb_ep_barrier)."""
    lib = _lib.load()
    with torch.cuda.device(my_pad.device):
        _lib.check(lib.sb_ep_barrier(_ptr(peer_pads), _ptr(my_pad), _ptr(epoch), my_rank, peer_pads.numel(),
                                     _ptr(status), _stream()))


# ---- dispatch overlapped with the owner's first matmul (see csrc/ep_dispatch.cuh) ----------------------

def ep_dispatch_segments(capacity: int) -> int:
    """Arrival flags (and the sender's chunk counters) per rank pair: one per 256 rows of the capacity."""
    return int(_lib.load().sb_ep_dispatch_segments(capacity))


def ep_owner_layout(recv_counts: torch.Tensor, capacity: int, ffn_dim: int, block_size: int = BLOCK,
                    arrival_order: bool = False) -> list[torch.Tensor]:
    """The owner's layout over its N * capacity receive slots from the exchanged counts [N, E_local] alone: the
    eight arrays build_topology_cuda returns for ep_slot_experts' output, in one launch (error always 0). With
    arrival_order a ninth array follows, the schedule ep_sdd_dispatch walks: the row blocks in the order their
    rows become complete when every source fills its slots from the front, then 64 ints per row block (how many
    arrival flags its rows depend on, and which)."""
    lib = _lib.load()
    _check(recv_counts.is_cuda and recv_counts.dtype == torch.int32 and recv_counts.dim() == 2 and
           recv_counts.is_contiguous(), "recv_counts must be a contiguous [N, E_local] int32 CUDA tensor")
    num_ranks, experts_local = recv_counts.shape
    n = num_ranks * capacity
    max_rb, max_rows, ffn_blocks = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _lib.check(lib.sb_route_sizes(n, experts_local, ffn_dim, block_size, ctypes.byref(max_rb), ctypes.byref(max_rows),
                                  ctypes.byref(ffn_blocks)))
    max_rb, max_rows, ffn_blocks = max_rb.value, max_rows.value, ffn_blocks.value
    with torch.cuda.device(recv_counts.device):
        sizes = [experts_local, experts_local + 1, max_rows, n, max_rb, max_rb + 1, max_rb * ffn_blocks, 1]
        if arrival_order:
            sizes.append(int(lib.sb_ep_dispatch_schedule_ints(max_rb)))
        parts = list(torch.split(torch.empty(sum(sizes), dtype=torch.int32, device=recv_counts.device), sizes))
        order = parts.pop() if arrival_order else None
        error = parts[7]
        _lib.check(lib.sb_ep_owner_layout(_ptr(recv_counts), num_ranks, experts_local, capacity, ffn_blocks, block_size,
                                          max_rb, *(_ptr(t) for t in parts[:7]), _ptr(order) if arrival_order else None,
                                          _ptr(error), _stream()))
    return parts + [order] if arrival_order else parts


def ep_push_rows_flagged(x: torch.Tensor, sorted_token: torch.Tensor, expert_offsets: torch.Tensor,
                         peer_recv: torch.Tensor, peer_flags: torch.Tensor, done: torch.Tensor, epoch: torch.Tensor,
                         my_rank: int, experts_per_rank: int, capacity: int) -> None:
    """The source side of the overlapped dispatch as a kernel of its own (sb_ep_push_rows_flagged)."""
    lib = _lib.load()
    _check(x.is_cuda and x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2-D CUDA tensor")
    _check_index(sorted_token, "sorted_token")
    _check_index(expert_offsets, "expert_offsets")
    num_ranks = peer_recv.numel()
    _check(expert_offsets.numel() == num_ranks * experts_per_rank + 1, "expert_offsets must have E + 1 entries")
    _check(done.numel() >= num_ranks * ep_dispatch_segments(capacity), "done needs one counter per (destination, segment)")
    with torch.cuda.device(x.device):
        _lib.check(lib.sb_ep_push_rows_flagged(_ptr(x), _ptr(sorted_token), _ptr(expert_offsets), _ptr(peer_recv),
                                               _ptr(peer_flags), _ptr(done), _ptr(epoch), my_rank, num_ranks,
                                               experts_per_rank, capacity, x.shape[1] * x.element_size(), _stream()))


def ep_sdd_dispatch(recv: torch.Tensor, w1: torch.Tensor, row_slot: torch.Tensor, row_block_expert: torch.Tensor,
                    row_offsets: torch.Tensor, num_nnz: int, x: torch.Tensor, sorted_token: torch.Tensor,
                    expert_offsets: torch.Tensor, row_block_order: torch.Tensor | None, peer_recv: torch.Tensor,
                    peer_flags: torch.Tensor, my_flags: torch.Tensor, done: torch.Tensor, epoch: torch.Tensor,
                    my_rank: int, capacity: int, push_warps: int = -1) -> torch.Tensor:
    """SDD + GELU over the receive buffer `recv` [N * capacity, D] whose rows are still arriving: extra warps of
    the same kernel push this rank's own rows `x[sorted_token]` to their owners, and every tile waits (bounded)
    for the 256-row segments its rows lie in. Tiles are walked in row_block_order (ep_owner_layout's arrival
    order; None: layout order). push_warps = 0: this rank's rows are pushed by ep_push_rows_flagged, launched before
    this call on another stream. Returns the blocks [num_nnz, 128, 128] like sdd_cuda with skip_padding_rows."""
    lib = _lib.load()
    _check(recv.is_cuda and w1.is_cuda and x.is_cuda and recv.device == w1.device == x.device, "all inputs on one GPU")
    _check(recv.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and x.dtype == torch.bfloat16, "rows and w1 must be bfloat16")
    _check(recv.is_contiguous() and w1.is_contiguous() and x.is_contiguous(), "recv, w1 and x must be contiguous")
    _check(recv.dim() == 2 and w1.dim() == 3 and x.dim() == 2 and w1.shape[1] == recv.shape[1] == x.shape[1],
           "recv and x must be [., D] and w1 [E_local, D, F]")
    for t, name in ((row_slot, "row_slot"), (row_block_expert, "row_block_expert"), (row_offsets, "row_offsets"),
                    (sorted_token, "sorted_token"), (expert_offsets, "expert_offsets")):
        _check_index(t, name)
    experts_local, d_model, ffn_dim = w1.shape
    num_ranks = peer_recv.numel()
    num_row_blocks = row_offsets.numel() - 1
    _check(recv.shape[0] == num_ranks * capacity, "recv must hold ranks * capacity rows")
    _check(d_model % 64 == 0 and ffn_dim % 256 == 0, "need D a multiple of 64 and F a multiple of 256")
    _check(row_slot.numel() == num_row_blocks * BLOCK and num_nnz == num_row_blocks * (ffn_dim // BLOCK),
           "the layout does not match block size 128")
    _check(expert_offsets.numel() == num_ranks * experts_local + 1, "expert_offsets must have E + 1 entries")
    if row_block_order is not None:
        _check_index(row_block_order, "row_block_order")
        _check(row_block_order.numel() == lib.sb_ep_dispatch_schedule_ints(num_row_blocks),
               "row_block_order must be ep_owner_layout's schedule for the same layout")
    segments = ep_dispatch_segments(capacity)
    _check(my_flags.numel() >= num_ranks * segments and done.numel() >= num_ranks * segments,
           "flags and counters need ranks * ep_dispatch_segments(capacity) entries")
    with torch.cuda.device(recv.device):
        out = torch.empty((num_nnz, BLOCK, BLOCK), dtype=torch.bfloat16, device=recv.device)
        _lib.check(lib.sb_ep_sdd_dispatch(_ptr(recv), _ptr(w1), _ptr(row_slot), _ptr(row_block_expert), _ptr(row_offsets),
                                          _ptr(out), d_model, ffn_dim, num_row_blocks, _ptr(x), _ptr(sorted_token),
                                          _ptr(expert_offsets), _ptr(row_block_order) if row_block_order is not None else None,
                                          _ptr(peer_recv), _ptr(peer_flags), _ptr(my_flags), _ptr(done),
                                          _ptr(epoch), my_rank, num_ranks, experts_local, capacity, push_warps,
                                          _ptr(device_status(recv.device)), _stream()))
    return out
