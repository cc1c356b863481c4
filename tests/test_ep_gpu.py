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
