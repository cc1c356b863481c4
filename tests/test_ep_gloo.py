"""The expert-parallel step on CPU ranks (gloo, world size 2 and 4): the orchestration of
sparsebench_b200/ep.py with the device operations replaced by the oracle-based stand-in of
tests/ep_cpu_ops.py. Checks, on every rank, that
  * the gathered outputs equal the single-process layer on the concatenated batch,
  * the owner's layout equals the single-process layout of the concatenated batch restricted to the
    owner's experts (global token id = rank*T + t), i.e. the exchange keeps the stable copy order,
  * a capacity that is too small raises the overflow flag instead of corrupting anything.
"""

import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import layout as L
from oracle import moe as M
from sparsebench_b200.workloads import routing_case

T, D, F, E, K = 48, 16, 128, 8, 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _global_batch(world: int, case: str):
    g = torch.Generator().manual_seed(11)
    x = torch.randn(world * T, D, generator=g)
    w1 = torch.randn(E, D, F, generator=g) / D**0.5
    w2 = torch.randn(E, F, D, generator=g) / F**0.5
    gate = torch.rand(world * T, K, generator=g)
    idx = routing_case(case, world * T, E, seed=5)
    return x, idx, gate, w1, w2


def _worker(rank: int, world: int, port: int, case: str, capacity: int | None) -> None:
    from sparsebench_b200.ep import ExpertParallelMoE, shard_experts
    from tests.ep_cpu_ops import CpuOps

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        x, idx, gate, w1, w2 = _global_batch(world, case)
        mine = slice(rank * T, (rank + 1) * T)
        layer = ExpertParallelMoE(shard_experts(w1, rank, world), shard_experts(w2, rank, world), E,
                                  capacity=capacity, ops=CpuOps())
        stages: list[str] = []
        out = layer(x[mine].contiguous(), idx[mine].contiguous(), gate[mine].contiguous(), mark=stages.append)
        assert stages == ["dispatch plan", "dispatch all-to-all", "routing", "SDD + GELU (fused)", "DSD",
                          "return all-to-all", "combine"]

        if capacity is not None and capacity < T * K:
            flags = [torch.zeros(1, dtype=torch.int32) for _ in range(world)]
            dist.all_gather(flags, layer.status)
            assert any(int(f) for f in flags), "a too-small capacity must raise the overflow flag somewhere"
            if int(layer.status) != 0:
                with pytest.raises(RuntimeError, match="capacity"):
                    layer.check()
            return
        layer.check()

        expected = M.moe_reference(x, idx, gate, w1, w2)[mine]
        torch.testing.assert_close(out, expected, rtol=1e-4, atol=1e-5)

        # Layout: owner's rows, expert by expert, against the single-process layout of the global batch.
        trace = layer.last
        cap = layer.capacity
        global_token = torch.where(trace.send_index >= 0, trace.send_index + rank * T, -1).to(torch.int32)
        received = torch.empty_like(global_token)
        dist.all_to_all_single(received, global_token)  # slot -> global token id of the copy in it
        whole = L.build_topology(idx, E, F, 128)
        per_rank = E // world
        owner = trace.owner_layout
        for e_local in range(per_rank):
            e = rank * per_rank + e_local
            count = int(whole.tokens_per_expert[e])
            assert int(owner.tokens_per_expert[e_local]) == count
            start_global, start_local = int(whole.padded_offsets[e]), int(owner.padded_offsets[e_local])
            slots = owner.row_token[start_local : start_local + count].long()
            assert np.array_equal(received[slots].numpy(), whole.row_token[start_global : start_global + count])
        assert world * cap == trace.slot_expert.numel()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize(("world", "case"), [(2, "random"), (2, "empty_middle"), (4, "zipf")])
def test_expert_parallel_step_matches_single_process(world: int, case: str) -> None:
    mp.spawn(_worker, args=(world, _free_port(), case, None), nprocs=world, join=True)


def test_small_capacity_raises_overflow_flag() -> None:
    mp.spawn(_worker, args=(2, _free_port(), "skewed", 8), nprocs=2, join=True)


def test_single_rank_is_the_plain_layer() -> None:
    # World size 1 without a process group: every all-to-all is the identity.
    from sparsebench_b200.ep import ExpertParallelMoE
    from tests.ep_cpu_ops import CpuOps

    x, idx, gate, w1, w2 = _global_batch(1, "zipf")
    out = ExpertParallelMoE(w1, w2, E, ops=CpuOps())(x, idx, gate)
    torch.testing.assert_close(out, M.moe_reference(x, idx, gate, w1, w2), rtol=1e-4, atol=1e-5)
