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

With the peer exchange the return leg rides inside the owner's DSD kernel, and the dispatch leg can ride
inside its SDD kernel (`fuse_dispatch`; otherwise one push kernel and a full barrier). Dispatch inside SDD: only the
per-expert COUNTS are exchanged up front (they are all the owner's layout needs); the rows are
pushed by extra warps of the SDD kernel itself, every destination's slots from the front, and every SDD
tile waits, bounded, for the arrival flags of the 256-row segments its rows lie in; the owner walks its
row blocks in the order they become complete, so the rows travel while the tensor cores already work
on what has arrived. Return: the DSD epilogue stores each result row into its source rank's buffer (no y, no
second kernel). Two device-side barriers remain per step: a light one after the counts, and the
one before the combine.

Slots arrive ordered by (source rank, expert, copy index), and the owner's sort is stable, so
within an expert rows follow (source rank, copy index): the global copy order with global token
id = rank*T + t. Concatenating the ranks' layouts therefore equals the single-GPU layout of the
concatenated batch, and the gathered outputs equal the single-GPU layer's.

Device work goes through an `ops` object so that the orchestration (and the exchange pattern) can
be exercised on CPU ranks with a stand-in from the tests; the default is the CUDA library.
"""

from __future__ import annotations

import math

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

        return sdd(x, w1, topo, gelu=True, skip_padding_rows=True)

    def dsd(self, h, w2_cat, topo):
        from sparsebench_b200.spmm import dsd

        return dsd(h, w2_cat, topo, version=5, skip_padding_rows=True)

    def combine(self, y: torch.Tensor, copy_row: torch.Tensor, expert_weight: torch.Tensor) -> torch.Tensor:
        from sparsebench_b200 import _C

        return _C.combine_cuda(y, copy_row, expert_weight)

    def push_rows(self, src, index, peer_base, my_rank, capacity) -> None:
        from sparsebench_b200 import _C

        _C.ep_push_rows(src, index, peer_base, my_rank, capacity)

    def push_counts(self, counts, peer_counts, my_rank, experts_per_rank) -> None:
        from sparsebench_b200 import _C

        _C.ep_push_counts(counts, peer_counts, my_rank, experts_per_rank)

    def dsd_push(self, h, w2_cat, topo, peer_base, my_rank, capacity) -> None:
        """dsd + push_rows of the result as one kernel: the DSD epilogue stores every row into the
        buffer of the rank it came from (topo.row_token is the owner's row -> receive slot table)."""
        from sparsebench_b200 import _C

        _C.ep_dsd_push(h, w2_cat, topo.row_offsets, topo.col_indices, topo.row_token, peer_base, my_rank, capacity)

    def barrier(self, peer_pads, my_pad, epoch, my_rank, status) -> None:
        from sparsebench_b200 import _C

        _C.ep_barrier(peer_pads, my_pad, epoch, my_rank, status)

    def owner_layout(self, recv_counts: torch.Tensor, capacity: int, ffn_dim: int, arrival_order: bool = False):
        """The owner's layout over its receive slots from the exchanged counts alone; with arrival_order, also the
        order in which its row blocks become complete (a second return value)."""
        from sparsebench_b200 import _C
        from sparsebench_b200.routing import DeviceTopology

        out = _C.ep_owner_layout(recv_counts, capacity, ffn_dim, BLOCK_SIZE, arrival_order)
        topo = DeviceTopology(BLOCK_SIZE, recv_counts.shape[1], ffn_dim // BLOCK_SIZE, *out[:8])
        return (topo, out[8]) if arrival_order else topo

    def sdd_dispatch(self, peer, w1, topo, order, x, sorted_token, expert_offsets, my_rank, capacity, push_warps=-1):
        """SDD over rows that are still arriving; this rank's own pushes run in the same kernel (push_warps != 0) or
        in a push_rows_flagged launched before it on another stream (push_warps = 0)."""
        from sparsebench_b200 import _C

        return _C.ep_sdd_dispatch(peer.recv, w1, topo.row_token, topo.row_block_expert, topo.row_offsets,
                                  topo.col_indices.numel(), x, sorted_token, expert_offsets, order, peer.peer_recv,
                                  peer.peer_flags, peer.flags, peer.done, peer.epoch, my_rank, capacity, push_warps)

    def push_rows_flagged(self, peer, x, sorted_token, expert_offsets, my_rank, experts_per_rank, capacity) -> None:
        """This rank's rows into their owners' receive buffers, one arrival flag per 256-row segment."""
        from sparsebench_b200 import _C

        _C.ep_push_rows_flagged(x, sorted_token, expert_offsets, peer.peer_recv, peer.peer_flags, peer.done, peer.epoch,
                                my_rank, experts_per_rank, capacity)


class PeerExchange:
    """Exchange buffers of one rank mapped into every other rank (torch symmetric memory: CUDA VMM
    handles exchanged once at set-up), so that rows are stored straight into their owner's memory
    over NVLink and only real rows travel. Holds, per rank: recv [N*C, D] (dispatched rows, block s
    from rank s), ret [N*C, D] (results coming back, block d from rank d), counts [N, E/N], a pad
    of N words for the device-side barrier and N * ceil(C / 256) arrival flags (one per source and 256-row
    segment of its block of recv)."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, capacity: int, d_model: int,
                 experts_local: int, dtype: torch.dtype = torch.bfloat16) -> None:
        import torch.distributed._symmetric_memory as symm

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        world = self.world
        elem = torch.empty(0, dtype=dtype).element_size()

        def aligned(n: int) -> int:
            return (n + 255) // 256 * 256

        rows_bytes = aligned(world * capacity * d_model * elem)
        counts_bytes = aligned(world * experts_local * 4)
        pad_bytes = aligned(world * 4)
        segments = (capacity + 255) // 256  # sb_ep_dispatch_segments
        flags_bytes = aligned(world * segments * 4)
        offsets = [0, rows_bytes, 2 * rows_bytes, 2 * rows_bytes + counts_bytes, 2 * rows_bytes + counts_bytes + pad_bytes]
        total = offsets[4] + flags_bytes
        self.buffer = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buffer, group)
        self.buffer[offsets[2]:].zero_()  # counts, barrier pad and arrival flags start at zero
        torch.cuda.synchronize(device)
        dist.barrier(group)

        def view(off: int, nbytes: int, dt: torch.dtype) -> torch.Tensor:
            return self.buffer[off : off + nbytes].view(dt)

        self.recv = view(offsets[0], world * capacity * d_model * elem, dtype).view(world * capacity, d_model)
        self.ret = view(offsets[1], world * capacity * d_model * elem, dtype).view(world * capacity, d_model)
        self.counts = view(offsets[2], world * experts_local * 4, torch.int32).view(world, experts_local)
        self.pad = view(offsets[3], world * 4, torch.int32)
        self.flags = view(offsets[4], world * segments * 4, torch.int32)
        bases = [int(p) for p in self.handle.buffer_ptrs]

        def table(off: int) -> torch.Tensor:
            return torch.tensor([b + off for b in bases], dtype=torch.int64, device=device)

        self.peer_recv, self.peer_ret = table(offsets[0]), table(offsets[1])
        self.peer_counts, self.peer_pads = table(offsets[2]), table(offsets[3])
        self.peer_flags = table(offsets[4])
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.done = torch.zeros(world * segments, dtype=torch.int32, device=device)  # push chunk counters


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
                 group: dist.ProcessGroup | None = None, capacity: int | None = None, ops: object | None = None,
                 exchange: str = "nccl", fuse_return: bool = True, micro_batches: int = 1,
                 fuse_dispatch: bool = False, push_beside: bool = True,
                 micro_fractions: tuple[float, ...] | None = None) -> None:
        """w1_local [E/N, D, F], w2_local [E/N, F, D]: this rank's experts. `capacity` = rows per
        (source, destination) pair; None means T*k of the first call's batch (never overflows).
        `exchange`: "nccl" = fixed-capacity all-to-all collectives (every slot travels, real or not);
        "peer" = rows stored straight into the owner's mapped memory by this library's kernels, with a
        device-side barrier (only real rows travel; needs `capacity` up front and world size > 1).
        `fuse_return` (peer exchange only): the owner's DSD stores its rows straight into the source
        ranks' buffers from its epilogue instead of writing y and pushing it with a second kernel.
        `fuse_dispatch` (peer exchange only): only the counts are exchanged before the owner's layout is
        built; the rows are pushed by extra warps of the owner's SDD kernel and every SDD tile waits for
        the segments its rows lie in, instead of pushing all rows and waiting for all ranks before SDD
        starts. `push_beside` (with fuse_dispatch): the rows are pushed by the stand-alone push kernel on a second
        stream, launched before the SDD kernel and running beside it (the whole GPU's warps push, the SDD tiles
        follow the arrivals), instead of by the SDD kernel's own six push warps per block.
        `micro_batches` (peer exchange only): the T local tokens are cut into that many equal parts, each
        a complete step with its own exchange buffers on its own stream, ordered so that part m+1 is
        dispatched while part m is computed and part m returns while part m+1 is computed. Same result
        bit for bit; every part reads the owner's expert weights again, so it pays only where the
        owner's matmuls are tensor-bound (many tokens per expert) and the exchange is a large share.
        `micro_fractions`: the parts' shares of the tokens instead of equal ones (one per micro-batch, summing
        to 1, the same on every rank): the first part's dispatch is the only one nothing hides, so a smaller
        first part shortens the step."""
        self.fuse_return = fuse_return
        self.fuse_dispatch = fuse_dispatch
        self.push_beside = push_beside
        self._push_streams: dict = {}
        self.micro_batches = int(micro_batches)
        if self.micro_batches < 1:
            raise ValueError("micro_batches must be >= 1")
        if micro_fractions is None:
            micro_fractions = tuple(1.0 / self.micro_batches for _ in range(self.micro_batches))
        if len(micro_fractions) != self.micro_batches or abs(sum(micro_fractions) - 1.0) > 1e-6 or \
                min(micro_fractions) <= 0.0:
            raise ValueError("micro_fractions needs one positive share per micro-batch, summing to 1")
        self.micro_fractions = tuple(float(f) for f in micro_fractions)
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
        self.status = torch.zeros(1, dtype=torch.int32, device=w1_local.device)  # sb_ep_status bits
        self.last: StepTrace | None = None
        if exchange not in ("nccl", "peer"):
            raise ValueError(f"exchange must be 'nccl' or 'peer', got {exchange!r}")
        self.peer: PeerExchange | None = None
        self.part_peers: list[PeerExchange] = []
        self.part_streams: list[torch.cuda.Stream] = []
        if exchange == "peer" and self.world > 1:
            if capacity is None:
                raise ValueError("the peer exchange sizes its buffers at construction: pass `capacity`")
            pg = group if group is not None else dist.group.WORLD
            if self.micro_batches == 1:
                self.peer = PeerExchange(pg, w1_local.device, capacity, d_model, experts_local, w1_local.dtype)
            else:
                # Every part gets its share of the capacity, rounded up to whole blocks of 128 rows plus one block
                # (the part boundaries are rounded to 8 tokens, so a part may hold a few rows more than its share).
                self.part_capacities = [min(capacity, -(-int(math.ceil(capacity * f)) // 128) * 128 + 128)
                                        for f in self.micro_fractions]
                for part_capacity in self.part_capacities:
                    self.part_peers.append(PeerExchange(pg, w1_local.device, part_capacity, d_model, experts_local,
                                                        w1_local.dtype))
                    self.part_streams.append(torch.cuda.Stream(device=w1_local.device))
                self.peer = self.part_peers[0]
        elif self.micro_batches != 1:
            raise ValueError("micro_batches needs the peer exchange and more than one rank")

    def _all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        """[N, ...] -> [N, ...]: block d goes to rank d, block s of the result came from rank s."""
        if self.world == 1:
            return send
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv

    def check(self) -> None:
        """Syncs. Raises if some (source, destination) run exceeded the capacity and copies were
        dropped, or if a device-side barrier gave up waiting for a peer."""
        status = int(self.status.item())
        if status & 2:
            raise RuntimeError("expert-parallel barrier timed out waiting for a peer rank")
        if status & 1:
            raise RuntimeError("expert-parallel exchange overflowed its capacity: raise `capacity`")

    def forward(self, x: torch.Tensor, expert_idx: torch.Tensor, expert_weight: torch.Tensor,
                mark: Callable[[str], None] = _no_mark) -> torch.Tensor:
        """x [T, D], expert_idx / expert_weight [T, k] with GLOBAL expert ids -> [T, D]. No host sync."""
        num_tokens, k = expert_idx.shape
        if x.shape != (num_tokens, self.d_model) or expert_weight.shape != expert_idx.shape:
            raise ValueError("x must be [T, D] and expert_idx / expert_weight [T, k]")
        if self.part_peers:
            return self._forward_pipelined(x, expert_idx, expert_weight, mark)
        return self._forward_part(x, expert_idx, expert_weight, mark, self.peer, self.capacity, None)

    def _forward_pipelined(self, x, expert_idx, expert_weight, mark) -> torch.Tensor:
        """The step as `micro_batches` independent part-steps on their own streams (forked from and
        joined back into the caller's stream, so it captures into one graph). Part m+1 may not start
        its dispatch before part m's rows have arrived (the two would only share the links), but
        does not wait for part m's matmuls: that is where the overlap comes from."""
        num_tokens = x.shape[0]
        # Part boundaries from the shares, on multiples of 8 tokens (the last part takes the remainder).
        bounds, running = [0], 0.0
        for f in self.micro_fractions[:-1]:
            running += f
            bounds.append(min(num_tokens, max(bounds[-1], int(round(running * num_tokens / 8.0)) * 8)))
        bounds.append(num_tokens)
        main = torch.cuda.current_stream()
        outs: list[torch.Tensor] = []
        dispatched: torch.cuda.Event | None = None
        for m, (peer, stream) in enumerate(zip(self.part_peers, self.part_streams)):
            rows = slice(bounds[m], bounds[m + 1])
            if rows.stop == rows.start:
                raise ValueError(f"{num_tokens} tokens leave micro-batch {m} empty with shares {self.micro_fractions}")
            stream.wait_stream(main)
            with torch.cuda.stream(stream):
                if dispatched is not None:
                    stream.wait_event(dispatched)
                arrived = torch.cuda.Event()
                out = self._forward_part(x[rows], expert_idx[rows], expert_weight[rows], mark if m == 0 else _no_mark,
                                         peer, self.part_capacities[m], arrived.record)
                out.record_stream(main)
            outs.append(out)
            dispatched = arrived
        for stream in self.part_streams:
            main.wait_stream(stream)
        return torch.cat(outs)

    def _forward_part(self, x, expert_idx, expert_weight, mark, peer, capacity, after_dispatch) -> torch.Tensor:
        num_tokens, k = expert_idx.shape
        n, world, ops = num_tokens * k, self.world, self.ops
        if capacity is None:
            capacity = self.capacity = n

        # 1-2. Sort local copies by global expert (no padding), plan the slots.
        counts, offsets, sorted_token, copy_pos = ops.sort_copies(expert_idx, self.num_experts)
        send_index, return_row = ops.plan(offsets, sorted_token, copy_pos, world, self.experts_local, capacity,
                                          self.status)
        mark("dispatch plan")
        if peer is not None and self.fuse_dispatch and hasattr(ops, "sdd_dispatch"):
            return self._forward_peer_overlapped(x, expert_weight, send_index, return_row, mark,
                                                 (counts, offsets, sorted_token, copy_pos), peer, capacity, after_dispatch)
        if peer is not None:
            return self._forward_peer(x, expert_weight, counts, send_index, return_row, mark,
                                      (counts, offsets, sorted_token, copy_pos), peer, capacity, after_dispatch)
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

    def _forward_peer(self, x, expert_weight, counts, send_index, return_row, mark, source_sort, peer, capacity,
                      after_dispatch) -> torch.Tensor:
        """Steps 3-5 with the rows stored directly into their owners' memory."""
        ops = self.ops
        ops.push_counts(counts, peer.peer_counts, self.rank, self.experts_local)
        ops.push_rows(x, send_index, peer.peer_recv, self.rank, capacity)
        ops.barrier(peer.peer_pads, peer.pad, peer.epoch, self.rank, self.status)
        if after_dispatch is not None:
            after_dispatch()
        mark("dispatch all-to-all")
        if hasattr(ops, "owner_layout"):
            # The owner's layout from the exchanged counts alone, one launch (the same arrays as slot experts +
            # routing over the N * C mostly empty receive slots).
            slot_expert = None
            topo = ops.owner_layout(peer.counts, capacity, self.ffn_dim)
        else:
            slot_expert = ops.slot_experts(peer.counts, capacity)
            topo = ops.route(slot_expert.view(-1, 1), self.experts_local, self.ffn_dim, BLOCK_SIZE)
        mark("routing")
        h = ops.sdd(peer.recv, self.w1, topo)
        mark("SDD + GELU (fused)")
        if self.fuse_return and hasattr(ops, "dsd_push"):
            # The DSD epilogue stores each row into its source rank's buffer: the return leg travels
            # over NVLink while the tensor cores work, and y never exists.
            ops.dsd_push(h, self.w2_cat, topo, peer.peer_ret, self.rank, capacity)
            mark("DSD")
        else:
            y = ops.dsd(h, self.w2_cat, topo)
            mark("DSD")
            ops.push_rows(y, topo.copy_row, peer.peer_ret, self.rank, capacity)
        ops.barrier(peer.peer_pads, peer.pad, peer.epoch, self.rank, self.status)
        mark("return all-to-all")
        out = ops.combine(peer.ret, return_row, expert_weight)
        mark("combine")
        self.last = StepTrace(source_sort, send_index, return_row, peer.counts, slot_expert, topo)
        return out

    def _forward_peer_overlapped(self, x, expert_weight, send_index, return_row, mark, source_sort, peer, capacity,
                                 after_dispatch) -> torch.Tensor:
        """Steps 3-5 with both exchange legs inside the owner's matmul kernels (see the module text)."""
        ops = self.ops
        _, offsets, sorted_token, _ = source_sort
        x = x.contiguous()
        counts = source_sort[0]
        ops.push_counts(counts, peer.peer_counts, self.rank, self.experts_local)
        ops.barrier(peer.peer_pads, peer.pad, peer.epoch, self.rank, self.status)  # counts only: nothing heavy to wait for
        mark("dispatch all-to-all")
        beside = self.push_beside and hasattr(ops, "push_rows_flagged")
        if beside:
            # The push kernel goes first, on a stream of its own: it waits for nothing, so it makes progress
            # whatever else is resident, and the SDD kernel launched after it finds rows arriving.
            main = torch.cuda.current_stream()
            side = self._push_streams.get(main)
            if side is None:
                side = self._push_streams[main] = torch.cuda.Stream(device=x.device)
            side.wait_stream(main)  # after the counts barrier: the epoch word carries this step's value
            with torch.cuda.stream(side):
                ops.push_rows_flagged(peer, x, sorted_token, offsets, self.rank, self.experts_local, capacity)
        topo, order = ops.owner_layout(peer.counts, capacity, self.ffn_dim, arrival_order=True)
        mark("routing")
        h = ops.sdd_dispatch(peer, self.w1, topo, order, x, sorted_token, offsets, self.rank, capacity,
                             0 if beside else -1)
        if beside:
            torch.cuda.current_stream().wait_stream(side)
        if after_dispatch is not None:
            after_dispatch()
        mark("SDD + GELU (fused)")
        if self.fuse_return and hasattr(ops, "dsd_push"):
            ops.dsd_push(h, self.w2_cat, topo, peer.peer_ret, self.rank, capacity)
            mark("DSD")
        else:
            y = ops.dsd(h, self.w2_cat, topo)
            mark("DSD")
            ops.push_rows(y, topo.copy_row, peer.peer_ret, self.rank, capacity)
        ops.barrier(peer.peer_pads, peer.pad, peer.epoch, self.rank, self.status)
        mark("return all-to-all")
        out = ops.combine(peer.ret, return_row, expert_weight)
        mark("combine")
        self.last = StepTrace(source_sort, send_index, return_row, peer.counts, None, topo)
        return out

    __call__ = forward


def shard_experts(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's contiguous slice of a [E, ...] expert-major weight tensor."""
    per_rank = w.shape[0] // world
    if per_rank * world != w.shape[0]:
        raise ValueError(f"{w.shape[0]} experts do not split evenly over {world} ranks")
    return w[rank * per_rank : (rank + 1) * per_rank].contiguous()
