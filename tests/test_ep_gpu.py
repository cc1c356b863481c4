"""Expert-parallel plumbing kernels and the whole expert-parallel step on one GPU (world size 1:
every all-to-all is the identity, every kernel of the step still runs). The multi-GPU run of the
same step is tests/ep_multi_gpu.py, launched by torchrun."""

import numpy as np
import pytest
import torch

from oracle import layout as L
from oracle import moe as M
from tests import ep_cpu_ops
from tests.cases import routing_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize(("num_tokens", "num_experts", "ranks", "capacity"),
                         [(300, 8, 2, 600), (300, 8, 4, 100), (4096, 128, 8, 8192), (20000, 64, 8, 40000)])
def test_sort_and_plan_match_the_restatement(num_tokens: int, num_experts: int, ranks: int, capacity: int) -> None:
    from sparsebench_b200 import _C

    idx = routing_case("zipf", num_tokens, num_experts, seed=3)
    counts, offsets, sorted_token, copy_pos, error = _C.sort_copies_cuda(idx.cuda(), num_experts)
    expected = L.device_layout(idx, num_experts, 1, 1)
    assert np.array_equal(counts.cpu().numpy(), expected.tokens_per_expert)
    assert np.array_equal(offsets.cpu().numpy(), expected.padded_offsets)
    assert np.array_equal(sorted_token.cpu().numpy(), expected.row_token)
    assert np.array_equal(copy_pos.cpu().numpy(), expected.copy_row)
    assert int(error.item()) == 0

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    per_rank = num_experts // ranks
    send_index, return_row = _C.ep_plan(offsets, sorted_token, copy_pos, ranks, per_rank, capacity, status)
    want_send, want_ret, want_overflow = ep_cpu_ops.plan(expected.padded_offsets, expected.row_token, expected.copy_row,
                                                         ranks, per_rank, capacity)
    assert np.array_equal(send_index.cpu().numpy(), want_send)
    assert np.array_equal(return_row.cpu().numpy(), want_ret)
    assert int(status.item()) == want_overflow


def test_slot_experts_matches_the_restatement() -> None:
    from sparsebench_b200 import _C

    g = torch.Generator().manual_seed(0)
    recv_counts = torch.randint(0, 40, (8, 16), generator=g, dtype=torch.int32)
    recv_counts[3] = 0  # a source that sent nothing
    for capacity in (64, 700):  # smaller and larger than what a source sent
        got = _C.ep_slot_experts(recv_counts.cuda(), capacity)
        assert np.array_equal(got.cpu().numpy(), ep_cpu_ops.slot_experts(recv_counts.numpy(), capacity))


def test_gather_rows_skips_negative_indices() -> None:
    from sparsebench_b200 import _C

    src = torch.randn(50, 264, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    index = torch.tensor([3, -1, 49, 0, -1, 3], dtype=torch.int32, device="cuda")
    out = torch.full((6, 264), 7.0, dtype=torch.bfloat16, device="cuda")
    _C.gather_rows(src, index, out)
    assert torch.equal(out[[0, 2, 3, 5]], src[[3, 49, 0, 3]])
    assert torch.all(out[[1, 4]] == 7.0)


@pytest.mark.parametrize("case", ["random", "zipf", "empty_middle"])
def test_single_rank_step_matches_oracle_and_plain_layer(case: str) -> None:
    from sparsebench_b200 import moe_forward
    from sparsebench_b200.ep import ExpertParallelMoE

    g = torch.Generator().manual_seed(2)
    num_tokens, num_experts, d_model, ffn_dim = 300, 16, 256, 512
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16()
    gate = torch.rand(num_tokens, 2, generator=g).bfloat16()
    idx = routing_case(case, num_tokens, num_experts)
    layer = ExpertParallelMoE(w1.cuda(), w2.cuda(), num_experts)
    out = layer(x.cuda(), idx.cuda(), gate.cuda())
    layer.check()
    expected = M.moe_reference(x.float(), idx, gate.float(), w1.float(), w2.float())
    torch.testing.assert_close(out.float().cpu(), expected, rtol=2e-2, atol=2e-2)
    # Same kernels on the same rows in the same order: bit-identical to the plain layer.
    assert torch.equal(out, moe_forward(x.cuda(), idx.cuda(), gate.cuda(), w1.cuda(), w2.cuda()))


def test_single_rank_step_in_a_cuda_graph() -> None:
    from sparsebench_b200.ep import ExpertParallelMoE
    from sparsebench_b200.workloads import LayerConfig, make_layer

    cfg = LayerConfig("t", 512, 256, 256, 16, "zipf")
    layer_in = make_layer(cfg).to("cuda")
    layer = ExpertParallelMoE(layer_in.w1, layer_in.w2, cfg.num_experts)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(layer_in.x, layer_in.expert_idx, layer_in.expert_weight)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer(layer_in.x, layer_in.expert_idx, layer_in.expert_weight)
    fresh = make_layer(cfg, token_seed=9)
    layer_in.x.copy_(fresh.x.cuda())
    layer_in.expert_idx.copy_(fresh.expert_idx.cuda())
    layer_in.expert_weight.copy_(fresh.expert_weight.cuda())
    graph.replay()
    torch.cuda.synchronize()
    expected = M.moe_reference(fresh.x.float(), fresh.expert_idx, fresh.expert_weight.float(), fresh.w1.float(),
                               fresh.w2.float())
    torch.testing.assert_close(out.float().cpu(), expected, rtol=2e-2, atol=2e-2)


def test_barrier_gives_up_with_a_status_instead_of_hanging() -> None:
    # Failure detection without a fault: a two-rank barrier whose "peer" (a second pad in this GPU's
    # own memory that nothing ever writes) never arrives. The wait is bounded: the kernel returns
    # after its limit with SB_EP_TIMEOUT in the status word, and the context stays usable.
    import time

    from sparsebench_b200 import _C

    pads = torch.zeros(2, 2, dtype=torch.int32, device="cuda")  # pads[r] = rank r's pad; we are rank 0
    peer_pads = torch.tensor([pads[0].data_ptr(), pads[1].data_ptr()], dtype=torch.int64, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    started = time.perf_counter()
    _C.ep_barrier(peer_pads, pads[0], epoch, 0, status)
    torch.cuda.synchronize()
    waited = time.perf_counter() - started
    assert int(status.item()) == 2, "SB_EP_TIMEOUT expected"
    assert 1.0 < waited < 10.0
    assert pads[0].tolist() == [1, 0] and pads[1].tolist() == [1, 0]  # we signalled both, rank 1 never did
    assert int(epoch.item()) == 1
    # The context is still healthy: a one-rank barrier completes at once.
    status.zero_()
    one = torch.tensor([pads[0].data_ptr()], dtype=torch.int64, device="cuda")
    _C.ep_barrier(one, pads[0], epoch, 0, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(epoch.item()) == 2


def test_push_rows_into_own_memory_matches_gather() -> None:
    # World size 1 view of the peer exchange: pushing through a "peer" table that points at this
    # GPU's own buffer must leave what the pack kernel leaves.
    from sparsebench_b200 import _C

    g = torch.Generator().manual_seed(4)
    src = torch.randn(100, 256, generator=g).bfloat16().cuda()
    index = torch.randint(-1, 100, (2 * 64,), generator=g, dtype=torch.int32).cuda()
    # Two "ranks" whose buffers are two halves of one tensor; we are rank 1 of 2, capacity 64.
    recv = torch.zeros(2, 2 * 64, 256, dtype=torch.bfloat16, device="cuda")
    table = torch.tensor([recv[0].data_ptr(), recv[1].data_ptr()], dtype=torch.int64, device="cuda")
    _C.ep_push_rows(src, index, table, 1, 64)
    torch.cuda.synchronize()
    packed = _C.gather_rows(src, index, torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda"))
    for peer in range(2):
        assert torch.equal(recv[peer, 64:128], packed[peer * 64:(peer + 1) * 64])  # rows land at [my_rank=1][i]
        assert torch.all(recv[peer, :64] == 0)


@pytest.mark.parametrize("case", ["zipf", "empty_middle"])
def test_dsd_push_into_own_memory_matches_dsd_then_push(case: str) -> None:
    # The fused return leg on one GPU: two "ranks" whose return buffers are two halves of one local
    # tensor. The rows the DSD epilogue stores must be the rows dsd + ep_push_rows leave, bit for bit,
    # and nothing else may be touched.
    from sparsebench_b200 import _C
    from sparsebench_b200.routing import route_device
    from sparsebench_b200.spmm import dsd, sdd
    from sparsebench_b200.workloads import routing_case

    ranks, capacity, experts, d_model, ffn_dim, my_rank = 2, 192, 4, 256, 512, 1
    g = torch.Generator().manual_seed(7)
    slots = ranks * capacity
    x = torch.randn(slots, d_model, generator=g).bfloat16().cuda()
    w1 = (torch.randn(experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16().cuda()
    w2 = (torch.randn(experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16().cuda()
    slot_expert = routing_case(case, slots, experts, seed=3)[:, :1].clone()
    slot_expert[torch.rand(slots, 1, generator=g) < 0.3] = -1  # empty receive slots
    topo = route_device(slot_expert.to(torch.int32).cuda(), experts, ffn_dim, 128)
    h = sdd(x, w1, topo, gelu=True, skip_padding_rows=True)
    w2_cat = w2.view(experts * ffn_dim, d_model)

    def buffers():
        ret = torch.full((ranks, ranks * capacity, d_model), 7.0, dtype=torch.bfloat16, device="cuda")
        return ret, torch.tensor([ret[r].data_ptr() for r in range(ranks)], dtype=torch.int64, device="cuda")

    want, table = buffers()
    y = dsd(h, w2_cat, topo, version=5, skip_padding_rows=True)
    _C.ep_push_rows(y, topo.copy_row, table, my_rank, capacity)
    got, table2 = buffers()
    _C.ep_dsd_push(h, w2_cat, topo.row_offsets, topo.col_indices, topo.row_token, table2, my_rank, capacity)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert bool((want != 7.0).any())


# ---- dispatch overlapped with the owner's first matmul ---------------------------------------------------

@pytest.mark.parametrize(("ranks", "experts_local", "capacity"), [(2, 4, 64), (8, 16, 8192), (4, 32, 300), (1, 8, 1000)])
def test_owner_layout_from_counts_equals_routing_of_the_slots(ranks: int, experts_local: int, capacity: int) -> None:
    # One launch from N * E_local counts must leave what slot experts + routing (k = 1) leave, bit for bit.
    from sparsebench_b200 import _C

    g = torch.Generator().manual_seed(ranks * 100 + experts_local)
    recv_counts = torch.randint(0, max(2, 2 * capacity // experts_local), (ranks, experts_local), generator=g,
                                dtype=torch.int32)
    recv_counts[0, 1:] = 0            # a source with a single expert
    recv_counts[-1] = 0               # a source that sent nothing
    recv_counts[:, experts_local // 2] = 0  # an expert nobody uses
    ffn_dim = 512
    got = _C.ep_owner_layout(recv_counts.cuda(), capacity, ffn_dim)
    slot_expert = _C.ep_slot_experts(recv_counts.cuda(), capacity)
    want = _C.build_topology_cuda(slot_expert.view(-1, 1), experts_local, ffn_dim, 128)
    names = ("tokens_per_expert", "padded_offsets", "row_token", "copy_row", "row_block_expert", "row_offsets", "col_indices")
    for name, a, b in zip(names, got, want):
        assert torch.equal(a, b), name
    assert int(got[-1].item()) == 0
    # And against the CPU oracle of the slot list.
    oracle = L.device_layout(torch.from_numpy(ep_cpu_ops.slot_experts(recv_counts.numpy(), capacity)).view(-1, 1),
                             experts_local, ffn_dim, 128)
    for name, a in zip(names, got):
        assert np.array_equal(a.cpu().numpy(), getattr(oracle, name)), name
    # The arrival order: same eight arrays, plus the row blocks sorted by their last-arriving slot.
    with_order = _C.ep_owner_layout(recv_counts.cuda(), capacity, ffn_dim, arrival_order=True)
    for name, a, b in zip(names, with_order, got):
        assert torch.equal(a, b), name
    want_order = ep_cpu_ops.arrival_order(oracle.row_token, capacity, 128)
    schedule = with_order[8].cpu().numpy()
    blocks = len(want_order)
    assert schedule.size == _C._lib.load().sb_ep_dispatch_schedule_ints(blocks) == blocks * 65
    assert np.array_equal(schedule[:blocks], want_order)
    assert sorted(want_order.tolist()) == list(range(blocks))
    lists = schedule[blocks:].reshape(blocks, 64)
    for rb, want in enumerate(ep_cpu_ops.arrival_waits(oracle.row_token, capacity, 128)):
        assert lists[rb, 0] == len(want) and lists[rb, 1: 1 + len(want)].tolist() == want, rb


def _C_segments(capacity: int) -> int:
    from sparsebench_b200 import _C

    segments = _C.ep_dispatch_segments(capacity)
    assert segments == (capacity + 255) // 256
    return segments


class LocalExchange:
    """The exchange buffers of `ranks` virtual ranks, all in this GPU's memory: what PeerExchange maps across
    GPUs, for tests that run one rank's kernels at a time (no two launches ever wait for each other)."""

    def __init__(self, ranks: int, capacity: int, d_model: int, experts_local: int) -> None:
        dev = "cuda"
        self.segments = _C_segments(capacity)
        self.recv = torch.zeros(ranks, ranks * capacity, d_model, dtype=torch.bfloat16, device=dev)
        self.ret = torch.zeros(ranks, ranks * capacity, d_model, dtype=torch.bfloat16, device=dev)
        self.counts = torch.zeros(ranks, ranks, experts_local, dtype=torch.int32, device=dev)
        self.pad = torch.zeros(ranks, ranks, dtype=torch.int32, device=dev)
        self.flags = torch.zeros(ranks, ranks * self.segments, dtype=torch.int32, device=dev)
        self.epoch = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(ranks)]
        self.done = [torch.zeros(ranks * self.segments, dtype=torch.int32, device=dev) for _ in range(ranks)]

        def table(t: torch.Tensor) -> torch.Tensor:
            return torch.tensor([t[r].data_ptr() for r in range(ranks)], dtype=torch.int64, device=dev)

        self.peer_recv, self.peer_ret = table(self.recv), table(self.ret)
        self.peer_counts, self.peer_pads, self.peer_flags = table(self.counts), table(self.pad), table(self.flags)

    def of(self, rank: int):
        """Rank `rank`'s view, with the attribute names of sparsebench_b200.ep.PeerExchange."""
        import types

        return types.SimpleNamespace(
            recv=self.recv[rank], ret=self.ret[rank], counts=self.counts[rank], pad=self.pad[rank], flags=self.flags[rank],
            epoch=self.epoch[rank], done=self.done[rank], peer_recv=self.peer_recv, peer_ret=self.peer_ret,
            peer_counts=self.peer_counts, peer_pads=self.peer_pads, peer_flags=self.peer_flags)


@pytest.mark.parametrize(("ranks", "capacity", "num_tokens"), [(2, 600, 300), (4, 40, 300), (2, 1024, 1500)])
def test_flagged_push_leaves_what_the_plain_push_leaves_and_raises_the_segment_flags(ranks: int, capacity: int,
                                                                                     num_tokens: int) -> None:
    from sparsebench_b200 import _C

    num_experts, d_model = 16, 256
    experts_local = num_experts // ranks
    g = torch.Generator().manual_seed(5)
    old, new = LocalExchange(ranks, capacity, d_model, experts_local), LocalExchange(ranks, capacity, d_model, experts_local)
    want_flags = torch.zeros(ranks, ranks * new.segments, dtype=torch.int32)
    for rank in range(ranks):  # one virtual rank at a time
        x = torch.randn(num_tokens, d_model, generator=g).bfloat16().cuda()
        idx = routing_case("zipf", num_tokens, num_experts, seed=rank).cuda()
        counts, offsets, sorted_token, copy_pos, _ = _C.sort_copies_cuda(idx, num_experts)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        send_index, _ = _C.ep_plan(offsets, sorted_token, copy_pos, ranks, experts_local, capacity, status)
        _C.ep_push_counts(counts, old.peer_counts, rank, experts_local)
        _C.ep_push_rows(x, send_index, old.peer_recv, rank, capacity)
        view = new.of(rank)
        view.epoch.fill_(7)
        _C.ep_push_counts(counts, new.peer_counts, rank, experts_local)
        _C.ep_push_rows_flagged(x, sorted_token, offsets, new.peer_recv, new.peer_flags, view.done, view.epoch, rank,
                                experts_local, capacity)
        torch.cuda.synchronize()
        assert int(view.done.abs().sum().item()) == 0, "chunk counters must be left at zero"
        raised = ep_cpu_ops.segment_flags(offsets.cpu().numpy(), ranks, experts_local, capacity)  # [d][g]
        assert int(ep_cpu_ops.kept_rows(offsets.cpu().numpy(), ranks, experts_local, capacity).sum()) == \
            int((send_index >= 0).sum().item())
        for d in range(ranks):
            want_flags[d, rank * new.segments: (rank + 1) * new.segments] = torch.from_numpy(raised[d]) * 7
    assert torch.equal(new.recv, old.recv)
    assert torch.equal(new.counts, old.counts)
    assert torch.equal(new.flags.cpu(), want_flags), "exactly the segments that hold rows carry the epoch"
    assert bool((want_flags == 7).any()) and (capacity < 256 or bool((want_flags == 0).any()))


PUSH_ENGINES = pytest.mark.parametrize("engine", ["0", "1"], ids=["push_warps", "bulk_copies"])


@PUSH_ENGINES
@pytest.mark.parametrize(("case", "d_model"), [("zipf", 256), ("random", 256), ("empty_middle", 256), ("zipf", 2048),
                                               ("random", 4096)])
def test_overlapped_dispatch_single_rank_is_the_plain_layer(case: str, d_model: int, engine: str, monkeypatch) -> None:
    # World size 1 with the exchange buffers in local memory: the SDD kernel pushes this rank's rows to
    # itself and waits for its own flags. Same rows, same kernels: bit-identical to moe_forward, in both
    # dispatch modes, eagerly and twice in a row (the second step must wait for the second epoch).
    from sparsebench_b200 import moe_forward
    from sparsebench_b200.ep import ExpertParallelMoE, _no_mark

    monkeypatch.setenv("SB_PUSH_ENGINE", engine)  # read at every launch: rows pushed by warps or by bulk copies
    g = torch.Generator().manual_seed(2)
    num_tokens, num_experts, ffn_dim = 300, 16, 512  # rows of 512 B, 4 KB and 8 KB: 4, 4 and 2 rows per bulk chunk
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16().cuda()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16().cuda()
    layer = ExpertParallelMoE(w1, w2, num_experts)
    capacity = num_tokens * 2
    peer = LocalExchange(1, capacity, d_model, num_experts).of(0)
    for step in range(2):
        x = torch.randn(num_tokens, d_model, generator=g).bfloat16().cuda()
        gate = torch.rand(num_tokens, 2, generator=g).bfloat16().cuda()
        idx = routing_case(case, num_tokens, num_experts, seed=step).cuda()
        want = moe_forward(x, idx, gate, w1, w2)
        # Overlapped with the push kernel beside the SDD kernel, overlapped with the SDD kernel's own pushes, separate.
        for overlapped, beside in ((True, True), (True, False), (False, False)):
            layer.fuse_dispatch, layer.push_beside = overlapped, beside
            out = layer._forward_part(x, idx, gate, _no_mark, peer, capacity, None)
            layer.check()
            assert torch.equal(out, want), f"step {step}, overlapped={overlapped}, beside={beside}"


@PUSH_ENGINES
def test_two_virtual_ranks_overlapped_dispatch_matches_oracle(engine: str, monkeypatch) -> None:
    # Two ranks' worth of data on one GPU, one rank's kernels at a time: rank 1's rows are pushed by the
    # stand-alone push kernel first (it waits for nothing), then rank 0's SDD pushes its own rows and finds
    # rank 1's flags already raised. Checks rank 0's SDD blocks against the oracle of the concatenated batch.
    from sparsebench_b200 import _C
    from sparsebench_b200.routing import DeviceTopology

    monkeypatch.setenv("SB_PUSH_ENGINE", engine)
    ranks, num_tokens, num_experts, d_model, ffn_dim = 2, 200, 8, 256, 512
    experts_local, capacity = num_experts // ranks, 400
    g = torch.Generator().manual_seed(9)
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    ex = LocalExchange(ranks, capacity, d_model, experts_local)
    xs = [torch.randn(num_tokens, d_model, generator=g).bfloat16() for _ in range(ranks)]
    idxs = [routing_case("random", num_tokens, num_experts, seed=10 + r) for r in range(ranks)]
    starts, sorts = [], []
    for rank in range(ranks):
        ex.epoch[rank].fill_(3)
        counts, offsets, sorted_token, _, _ = _C.sort_copies_cuda(idxs[rank].cuda(), num_experts)
        _C.ep_push_counts(counts, ex.peer_counts, rank, experts_local)
        starts.append(offsets)
        sorts.append(sorted_token)
    x_dev = [x.cuda() for x in xs]
    view1 = ex.of(1)
    _C.ep_push_rows_flagged(x_dev[1], sorts[1], starts[1], ex.peer_recv, ex.peer_flags, view1.done, view1.epoch, 1,
                            experts_local, capacity)
    torch.cuda.synchronize()
    view0 = ex.of(0)
    *out, order = _C.ep_owner_layout(view0.counts, capacity, ffn_dim, arrival_order=True)
    topo = DeviceTopology(128, experts_local, ffn_dim // 128, *out)
    h = _C.ep_sdd_dispatch(view0.recv, w1[:experts_local].cuda(), topo.row_token, topo.row_block_expert, topo.row_offsets,
                           topo.col_indices.numel(), x_dev[0], sorts[0], starts[0], order, ex.peer_recv, ex.peer_flags,
                           view0.flags, view0.done, view0.epoch, 0, capacity)
    torch.cuda.synchronize()
    # Oracle: rank 0 owns experts [0, experts_local); its rows are the global batch's rows of those experts.
    x_all, idx_all = torch.cat(xs), torch.cat(idxs)
    whole = L.build_topology(idx_all, num_experts, ffn_dim, 128)
    blocks = M.sdd_blocks(x_all.float(), w1.float(), whole, gelu=True)
    rows_owned = int(whole.padded_offsets[experts_local])
    live = rows_owned // 128 * (ffn_dim // 128)
    counts = whole.tokens_per_expert[:experts_local]
    got, want = h[:live].float().cpu().view(-1, ffn_dim // 128, 128, 128), blocks[:live].view(-1, ffn_dim // 128, 128, 128)
    for e in range(experts_local):  # compare each expert's real rows (padding groups of 32 are not stored)
        first_rb = int(whole.padded_offsets[e]) // 128
        for j in range(int(counts[e])):
            rb, r = first_rb + j // 128, j % 128
            torch.testing.assert_close(got[rb, :, r], want[rb, :, r], rtol=1.6e-2, atol=1.6e-2)


@PUSH_ENGINES
def test_overlapped_dispatch_gives_up_with_a_status_when_a_source_never_delivers(engine: str, monkeypatch) -> None:
    # Failure detection without a fault: two virtual ranks, rank 1 never pushes, so its arrival flags are
    # never raised. Rank 0's SDD waits its bounded second per tile role, records SB_DEV_TIMEOUT_DISPATCH in
    # the status word and winds down; the context stays usable.
    import time

    from sparsebench_b200 import _C
    from sparsebench_b200.routing import DeviceTopology

    monkeypatch.setenv("SB_PUSH_ENGINE", engine)
    ranks, num_tokens, num_experts, d_model, ffn_dim, capacity = 2, 64, 4, 256, 256, 128
    experts_local = num_experts // ranks
    g = torch.Generator().manual_seed(1)
    ex = LocalExchange(ranks, capacity, d_model, experts_local)
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16().cuda()
    w1 = torch.randn(experts_local, d_model, ffn_dim, generator=g).bfloat16().cuda()
    idx = routing_case("random", num_tokens, num_experts, seed=0).cuda()
    counts, offsets, sorted_token, _, _ = _C.sort_copies_cuda(idx, num_experts)
    view = ex.of(0)
    view.epoch.fill_(1)
    _C.ep_push_counts(counts, ex.peer_counts, 0, experts_local)
    view.counts[1] = view.counts[0]  # pretend rank 1 announced rows that never come
    topo = DeviceTopology(128, experts_local, ffn_dim // 128, *_C.ep_owner_layout(view.counts, capacity, ffn_dim))
    status = _C.device_status(torch.device("cuda", torch.cuda.current_device()))
    torch.cuda.synchronize()
    started = time.perf_counter()
    _C.ep_sdd_dispatch(view.recv, w1, topo.row_token, topo.row_block_expert, topo.row_offsets, topo.col_indices.numel(),
                       x, sorted_token, offsets, None, ex.peer_recv, ex.peer_flags, view.flags, view.done, view.epoch, 0,
                       capacity)
    torch.cuda.synchronize()
    waited = time.perf_counter() - started
    word = int(status.item())
    status.zero_()
    assert word & 8, f"SB_DEV_TIMEOUT_DISPATCH expected in the status word, got {word}"
    assert 0.5 < waited < 20.0
    assert ex.flags[0].tolist() == [1, 0], "rank 0's own segment arrived, rank 1's never did"
    # Still healthy: the plain kernel runs.
    assert int(_C.arch_probe(4)[0].item()) == 1000
