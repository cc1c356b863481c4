"""CPU stand-in for the device operations of an expert-parallel step. TEST INFRASTRUCTURE.

Lets the orchestration in sparsebench_b200/ep.py (slot planning, the three all-to-alls, the owner's
layer over its receive slots) run on CPU ranks under gloo. Every operation is restated with the
oracle or plain numpy, following what the CUDA entry points document in
include/sparsebench_b200.h; the product never imports this file.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from oracle import layout as L
from oracle import moe as M
from sparsebench_b200.routing import DeviceTopology


def _t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))


def trimmed(dev: L.Layout) -> L.Layout:
    """The real-size view of a worst-case device layout."""
    rows = int(dev.padded_offsets[-1])
    rbs = rows // dev.block_size
    return dataclasses.replace(
        dev, row_token=dev.row_token[:rows], row_block_expert=dev.row_block_expert[:rbs],
        row_offsets=dev.row_offsets[: rbs + 1], col_indices=dev.col_indices[: rbs * dev.ffn_blocks])


def plan(offsets: np.ndarray, sorted_token: np.ndarray, copy_pos: np.ndarray, num_ranks: int, experts_per_rank: int,
         capacity: int) -> tuple[np.ndarray, np.ndarray, int]:
    """numpy restatement of sb_ep_plan: (send_index [N*C], return_row [n], overflow flag)."""
    starts = offsets[::experts_per_rank][: num_ranks + 1].astype(np.int64)
    send_index = np.full(num_ranks * capacity, -1, dtype=np.int32)
    overflow = 0
    for d in range(num_ranks):
        cnt = int(starts[d + 1] - starts[d])
        take = min(cnt, capacity)
        send_index[d * capacity : d * capacity + take] = sorted_token[starts[d] : starts[d] + take]
        overflow |= int(cnt > capacity)
    return_row = np.full(copy_pos.shape[0], -1, dtype=np.int32)
    for c, pos in enumerate(copy_pos):
        if pos < 0:
            continue
        d = int(np.searchsorted(starts[1:], pos, side="right"))
        i = int(pos - starts[d])
        if i < capacity:
            return_row[c] = d * capacity + i
    return send_index, return_row, overflow


def slot_experts(recv_counts: np.ndarray, capacity: int) -> np.ndarray:
    """numpy restatement of sb_ep_slot_experts."""
    num_ranks, experts_per_rank = recv_counts.shape
    out = np.full(num_ranks * capacity, -1, dtype=np.int32)
    for s in range(num_ranks):
        ids = np.repeat(np.arange(experts_per_rank, dtype=np.int32), np.maximum(recv_counts[s], 0))[:capacity]
        out[s * capacity : s * capacity + ids.shape[0]] = ids
    return out


class CpuOps:
    """Same method names and meanings as sparsebench_b200.ep.CudaOps, on CPU tensors."""

    def sort_copies(self, expert_idx: torch.Tensor, num_experts: int):
        dev = L.device_layout(expert_idx, num_experts, 1, 1)
        return _t(dev.tokens_per_expert), _t(dev.padded_offsets), _t(dev.row_token), _t(dev.copy_row)

    def plan(self, offsets, sorted_token, copy_pos, num_ranks, experts_per_rank, capacity, status):
        send_index, return_row, overflow = plan(offsets.numpy(), sorted_token.numpy(), copy_pos.numpy(), num_ranks,
                                                experts_per_rank, capacity)
        status |= overflow
        return _t(send_index), _t(return_row)

    def slot_experts(self, recv_counts: torch.Tensor, capacity: int) -> torch.Tensor:
        return _t(slot_experts(recv_counts.numpy(), capacity))

    def gather_rows(self, src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(index.numel(), src.shape[1], dtype=src.dtype)
        keep = index >= 0
        out[keep] = src[index[keep].long()]
        return out

    def route(self, expert_idx: torch.Tensor, num_experts: int, ffn_dim: int, block_size: int) -> DeviceTopology:
        dev = L.device_layout(expert_idx, num_experts, ffn_dim, block_size)
        self._layout = trimmed(dev)
        fields = {f: _t(getattr(dev, f)) for f in L.Layout.FIELDS}
        return DeviceTopology(block_size, num_experts, dev.ffn_blocks, error=torch.tensor([dev.error], dtype=torch.int32),
                              **fields)

    def sdd(self, x: torch.Tensor, w1: torch.Tensor, topo: DeviceTopology) -> torch.Tensor:
        live = M.sdd_blocks(x.float(), w1.float(), self._layout, gelu=True)
        out = torch.zeros(topo.col_indices.numel(), 128, 128)
        out[: live.shape[0]] = live
        return out

    def dsd(self, h: torch.Tensor, w2_cat: torch.Tensor, topo: DeviceTopology) -> torch.Tensor:
        live = M.dsd_rows(h[: self._layout.nnz_blocks], w2_cat.float(), self._layout)
        out = torch.zeros(topo.row_token.numel(), w2_cat.shape[1])
        out[: live.shape[0]] = live
        return out

    def combine(self, y: torch.Tensor, copy_row: torch.Tensor, expert_weight: torch.Tensor) -> torch.Tensor:
        num_tokens, k = expert_weight.shape
        rows = y[copy_row.long().clamp(min=0)].view(num_tokens, k, -1)
        rows = rows * (copy_row >= 0).view(num_tokens, k, 1)
        return (rows.float() * expert_weight.float()[..., None]).sum(dim=1)


def kept_rows(offsets: np.ndarray, num_ranks: int, experts_per_rank: int, capacity: int) -> np.ndarray:
    """Rows a source pushes to every destination d: its copies for d's experts, cut at the capacity."""
    starts = offsets[:: experts_per_rank][: num_ranks + 1].astype(np.int64)
    return np.minimum(capacity, starts[1:] - starts[:-1])


def segment_flags(offsets: np.ndarray, num_ranks: int, experts_per_rank: int, capacity: int,
                  segment_rows: int = 256) -> np.ndarray:
    """numpy restatement of which arrival flags a source raises (sb_ep_push_rows_flagged): [d][g] = 1 when segment g
    (slots g * 256 ...) of its block at destination d holds at least one row."""
    segments = -(-capacity // segment_rows)
    kept = kept_rows(offsets, num_ranks, experts_per_rank, capacity)
    return (kept[:, None] > np.arange(segments)[None, :] * segment_rows).astype(np.int32)


def arrival_order(row_token: np.ndarray, capacity: int, block_size: int) -> np.ndarray:
    """numpy restatement of sb_ep_owner_layout's row_block_order: row blocks sorted by the largest slot index
    (within its source's block of `capacity` slots) among their rows; ties in layout order, blocks without rows last."""
    rows = np.asarray(row_token, dtype=np.int64).reshape(-1, block_size)
    within = np.where(rows >= 0, rows % capacity, -1)
    keys = np.where((rows >= 0).any(axis=1), within.max(axis=1), np.iinfo(np.int32).max)
    return np.argsort(keys, kind="stable").astype(np.int32)


def arrival_waits(row_token: np.ndarray, capacity: int, block_size: int, segment_rows: int = 256) -> list[list[int]]:
    """numpy restatement of the wait lists in sb_ep_owner_layout's schedule: per row block the arrival flags
    (source * segments + segment) its rows lie in, sources ascending, segments ascending within a source."""
    segments = -(-capacity // segment_rows)
    lists = []
    for rows in np.asarray(row_token, dtype=np.int64).reshape(-1, block_size):
        real = rows[rows >= 0]
        source, within = real // capacity, real % capacity
        flags: list[int] = []
        for src in np.unique(source):
            slots = within[source == src]
            flags.extend(int(src) * segments + g for g in range(int(slots.min()) // segment_rows, int(slots.max()) // segment_rows + 1))
        lists.append(flags)
    return lists
