"""Expert-parallel MoE forward: experts sharded over the GPUs of one box, tokens exchanged by
all-to-all, every rank's step free of host syncs.

The reference is single-GPU; this mode reuses its four stages unchanged on each rank and adds one
exchange each way. With N ranks and E experts, rank d holds experts [d*E/N, (d+1)*E/N) (its
slices of w1/w2 never move) and T local tokens. One step on a rank:

  1. sort the T*k local copies by GLOBAL expert id (the routing kernel at block size 1: no
     padding), which makes the copies bound for rank d one contiguous run;
  2. plan: which token fills send slot (d, i), in which slot each copy's result will come back;
  3. pack the send buffer [N, C, D] (gather of token rows) and exchange it, together with the
     per-expert counts [N, E/N], by all-to-all. C rows per (source, destination) pair is a fixed
     capacity, so nothing depends on a count the host does not know (C = T*k is always exact;
     a smaller C trades traffic for an overflow flag);
  4. the owner derives the local expert of every receive slot from the counts, runs routing
     (k = 1, empty slots skipped), SDD and DSD on the received rows exactly as on one GPU;
  5. pack each slot's result row, exchange back, and combine with the local gates.

Slots arrive ordered by (source rank, expert, copy index), and the owner's sort is stable, so
within an expert rows follow (source rank, copy index): the global copy order with global token
id = rank*T + t. Concatenating the ranks' layouts therefore equals the single-GPU layout of the
concatenated batch, and the gathered outputs equal the single-GPU layer's.

Device work goes through an `ops` object so that the orchestration (and the exchange pattern) can
be exercised on CPU ranks with a stand-in from the tests; the default is the CUDA library.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass

import torch
import torch.distributed as dist

BLOCK_SIZE = 128


def _no_mark(stage: str) -> None:
    pass


class CudaOps:
    """The device operations of one step, served by libsparsebench_b200 (no fallback)."""

    def route(self, expert_idx: torch.Tensor, num_experts: int, ffn_dim: int, block_size: int):
        from sparsebench_b200.routing import route_device

        return route_device(expert_idx, num_experts, ffn_dim, block_size)

    def sort_copies(self, expert_idx: torch.Tensor, num_experts: int):
        """-> (tokens_per_expert [E], offsets [E+1], sorted_token [n], copy_pos [n])"""
        from sparsebench_b200 import _C

        return _C.sort_copies_cuda(expert_idx, num_experts)[:4]

    def plan(self, expert_offsets, sorted_token, copy_pos, num_ranks, experts_per_rank, capacity, status):
        from sparsebench_b200 import _C

        return _C.ep_plan(expert_offsets, sorted_token, copy_pos, num_ranks, experts_per_rank, capacity, status)

    def slot_experts(self, recv_counts: torch.Tensor, capacity: int) -> torch.Tensor:
        from sparsebench_b200 import _C

        return _C.ep_slot_experts(recv_counts, capacity)

    def gather_rows(self, src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
        from sparsebench_b200 import _C

        return _C.gather_rows(src, index)

    def sdd(self, x, w1, topo):
        from sparsebench_b200.spmm import sdd

        return sdd(x, w1, topo, gelu=True)

    def dsd(self, h, w2_cat, topo):
        from sparsebench_b200.spmm import dsd

        return dsd(h, w2_cat, topo, version=5)

    def combine(self, y: torch.Tensor, copy_row: torch.Tensor, expert_weight: torch.Tensor) -> torch.Tensor:
        from sparsebench_b200 import _C

        return _C.combine_cuda(y, copy_row, expert_weight)


@dataclass
class StepTrace:
    """What a step leaves behind for tests and debugging (device tensors; reading them syncs)."""

    source_sort: tuple  # (counts, offsets, sorted_token, copy_pos) of the local sort by global expert
    send_index: torch.Tensor  # [N*C]
    return_row: torch.Tensor  # [T*k]
    recv_counts: torch.Tensor  # [N, E/N]
    slot_expert: torch.Tensor  # [N*C]
    owner_layout: object  # the owner's DeviceTopology over its receive slots


class ExpertParallelMoE:
    """One rank's share of an expert-parallel layer."""

    def __init__(self, w1_local: torch.Tensor, w2_local: torch.Tensor, num_experts: int,
                 group: dist.ProcessGroup | None = None, capacity: int | None = None, ops: object | None = None) -> None:
        """w1_local [E/N, D, F], w2_local [E/N, F, D]: this rank's experts. `capacity` = rows per
        (source, destination) pair; None means T*k of the first call's batch (never overflows)."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        experts_local, d_model, ffn_dim = w1_local.shape
        if w2_local.shape != (experts_local, ffn_dim, d_model):
            raise ValueError(f"w2_local must be {(experts_local, ffn_dim, d_model)}, got {tuple(w2_local.shape)}")
        if experts_local * self.world != num_experts:
            raise ValueError(f"{num_experts} experts do not split into {self.world} ranks of {experts_local}")
        self.w1, self.w2_cat = w1_local, w2_local.view(experts_local * ffn_dim, d_model)
        self.num_experts, self.experts_local, self.d_model, self.ffn_dim = num_experts, experts_local, d_model, ffn_dim
        self.capacity = capacity
        self.ops = ops if ops is not None else CudaOps()
        self.status = torch.zeros(1, dtype=torch.int32, device=w1_local.device)  # SB_EP_OVERFLOW bits
        self.last: StepTrace | None = None

    def _all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        """[N, ...] -> [N, ...]: block d goes to rank d, block s of the result came from rank s."""
        if self.world == 1:
            return send
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv

    def check(self) -> None:
        """Syncs. Raises if some (source, destination) run exceeded the capacity and copies were dropped."""
        if int(self.status.item()) != 0:
            raise RuntimeError("expert-parallel exchange overflowed its capacity: raise `capacity`")

    def forward(self, x: torch.Tensor, expert_idx: torch.Tensor, expert_weight: torch.Tensor,
                mark: Callable[[str], None] = _no_mark) -> torch.Tensor:
        """x [T, D], expert_idx / expert_weight [T, k] with GLOBAL expert ids -> [T, D]. No host sync."""
        num_tokens, k = expert_idx.shape
        if x.shape != (num_tokens, self.d_model) or expert_weight.shape != expert_idx.shape:
            raise ValueError("x must be [T, D] and expert_idx / expert_weight [T, k]")
        n, world, ops = num_tokens * k, self.world, self.ops
        if self.capacity is None:
            self.capacity = n
        capacity = self.capacity

        # 1-2. Sort local copies by global expert (no padding), plan the slots.
        counts, offsets, sorted_token, copy_pos = ops.sort_copies(expert_idx, self.num_experts)
        send_index, return_row = ops.plan(offsets, sorted_token, copy_pos, world, self.experts_local, capacity,
                                          self.status)
        mark("dispatch plan")
        # 3. Pack and exchange rows and counts.
        send = ops.gather_rows(x, send_index)  # [N*C, D]; rows of empty slots are never read
        recv_counts = self._all_to_all(counts.view(world, self.experts_local))
        recv = self._all_to_all(send.view(world, capacity, self.d_model)).view(world * capacity, self.d_model)
        mark("dispatch all-to-all")
        # 4. The owner's layer over its receive slots (k = 1: a slot is a token).
        slot_expert = ops.slot_experts(recv_counts, capacity)
        topo = ops.route(slot_expert.view(-1, 1), self.experts_local, self.ffn_dim, BLOCK_SIZE)
        mark("routing")
        h = ops.sdd(recv, self.w1, topo)
        mark("SDD + GELU (fused)")
        y = ops.dsd(h, self.w2_cat, topo)
        mark("DSD")
        # 5. Results back to their sources, then the local gate-weighted sum.
        back = ops.gather_rows(y, topo.copy_row)  # [N*C, D] in slot order
        returned = self._all_to_all(back.view(world, capacity, self.d_model)).view(world * capacity, self.d_model)
        mark("return all-to-all")
        out = ops.combine(returned, return_row, expert_weight)
        mark("combine")
        self.last = StepTrace((counts, offsets, sorted_token, copy_pos), send_index, return_row, recv_counts, slot_expert, topo)
        return out

    __call__ = forward


def shard_experts(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's contiguous slice of a [E, ...] expert-major weight tensor."""
    per_rank = w.shape[0] // world
    if per_rank * world != w.shape[0]:
        raise ValueError(f"{w.shape[0]} experts do not split evenly over {world} ranks")
    return w[rank * per_rank : (rank + 1) * per_rank].contiguous()
