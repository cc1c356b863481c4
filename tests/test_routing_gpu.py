"""Routing on the GPU must reproduce the CPU layout bit for bit (reference: tests/test_routing.py)."""

import numpy as np
import pytest
import torch

from oracle import layout as L
from tests.cases import CASE_NAMES, FIELDS, assert_layout_equal, digest, load_golden, random_topk, routing_case

pytestmark = pytest.mark.gpu


def route_cuda(expert_idx: torch.Tensor, num_experts: int, ffn_dim: int, block_size: int):
    from sparsebench_b200.routing import build_topology_cuda

    return build_topology_cuda(expert_idx, num_experts, ffn_dim, block_size)


def check_against_oracle(expert_idx: torch.Tensor, num_experts: int, block_size: int) -> None:
    ffn_dim = 2 * block_size
    expected = L.build_topology(expert_idx, num_experts, ffn_dim, block_size)
    assert_layout_equal(route_cuda(expert_idx.cuda(), num_experts, ffn_dim, block_size), expected)


def check_device_buffers(expert_idx: torch.Tensor, num_experts: int, ffn_dim: int, block_size: int) -> None:
    """Every worst-case buffer, tails and error flag included."""
    from sparsebench_b200.routing import route_device

    dev = route_device(expert_idx.cuda(), num_experts, ffn_dim, block_size)
    expected = L.device_layout(expert_idx, num_experts, ffn_dim, block_size)
    for f in FIELDS:
        assert np.array_equal(getattr(dev, f).cpu().numpy(), getattr(expected, f)), f
    assert int(dev.error.item()) == expected.error


# Token counts hit: 1 copy per choice, not a multiple of 32, crosses a warp run, many runs.
@pytest.mark.parametrize("case", CASE_NAMES)
@pytest.mark.parametrize("num_experts", [2, 8, 64, 256])
@pytest.mark.parametrize("block_size", [4, 16, 128])
@pytest.mark.parametrize("num_tokens", [1, 13, 129, 1000])
def test_matches_oracle(case: str, num_experts: int, block_size: int, num_tokens: int) -> None:
    check_against_oracle(routing_case(case, num_tokens, num_experts), num_experts, block_size)


@pytest.mark.parametrize("k", [1, 2, 4])
@pytest.mark.parametrize("num_tokens", [1, 77, 3000])
def test_matches_oracle_any_k(k: int, num_tokens: int) -> None:
    check_against_oracle(random_topk(num_tokens, 16, k), 16, 16)


@pytest.mark.parametrize("case", ["random", "skewed"])
@pytest.mark.parametrize("num_experts", [8, 1024])
def test_matches_oracle_big(case: str, num_experts: int) -> None:
    # 200k copies (the largest cluster shape) and 320k copies (the three-launch shape with scratch).
    check_against_oracle(routing_case(case, 100_000, num_experts), num_experts, 128)
    check_against_oracle(routing_case(case, 160_000, num_experts), num_experts, 128)


@pytest.mark.parametrize("num_tokens", [511, 512, 513, 4097, 16385, 40000, 65535, 65536, 65537, 131072, 150_000])
def test_both_launch_shapes_around_their_switches(num_tokens: int) -> None:
    # Cluster of 1..8 blocks, 1/4/16 steps per warp; 131072 copies (65536 tokens here) is the last size the
    # single-launch cluster shape takes, beyond it the three-launch shape with scratch runs.
    idx = routing_case("random", num_tokens, 128)
    check_device_buffers(idx, 128, 512, 128)


@pytest.mark.parametrize("num_experts", [1, 2, 3, 5, 127, 129, 1000, 1024])
def test_expert_counts_that_are_not_powers_of_two(num_experts: int) -> None:
    # The peer mask is built from ceil(log2(E)) ballots: cover the edges of that count.
    k = min(2, num_experts)
    idx = random_topk(3000, num_experts, k)
    check_device_buffers(idx, num_experts, 256, 128)


@pytest.mark.parametrize("tag", [str(n) for n in load_golden("topology_cases.npz")["names"]])
def test_matches_reference_golden(tag: str) -> None:
    g = load_golden("topology_cases.npz")
    num_experts, ffn_dim, bs, full = (int(v) for v in g[f"{tag}/meta"])
    if full:
        got = route_cuda(torch.from_numpy(g[f"{tag}/expert_idx"]).cuda(), num_experts, ffn_dim, bs)
        for f in FIELDS:
            assert np.array_equal(getattr(got, f).cpu().numpy(), g[f"{tag}/{f}"]), f
    else:
        case, t, e, _ = tag.split("-")
        got = route_cuda(routing_case(case, int(t[1:]), int(e[1:])).cuda(), num_experts, ffn_dim, bs)
        assert [digest(getattr(got, f).cpu().numpy()) for f in FIELDS] == [str(d) for d in g[f"{tag}/digests"]]


@pytest.mark.parametrize("name", ["fine_grained", "fine_grained_zipf", "mixtral_like", "expert_parallel"])
def test_benchmark_configurations_full_size(name: str) -> None:
    from sparsebench_b200.workloads import CONFIGS

    cfg = CONFIGS[name]
    idx = routing_case(cfg.routing, cfg.num_tokens, cfg.num_experts)
    check_device_buffers(idx, cfg.num_experts, cfg.ffn_dim, 128)


def test_int32_and_int64_input_agree() -> None:
    idx = routing_case("random", 500, 8).cuda()
    a, b = route_cuda(idx.int(), 8, 32, 16), route_cuda(idx, 8, 32, 16)
    for f in FIELDS:
        assert torch.equal(getattr(a, f), getattr(b, f)), f


def test_deterministic() -> None:
    idx = routing_case("skewed", 5000, 64).cuda()
    a, b = route_cuda(idx, 64, 256, 128), route_cuda(idx, 64, 256, 128)
    for f in FIELDS:
        assert torch.equal(getattr(a, f), getattr(b, f)), f


def test_worst_case_buffers_are_marked_past_the_end() -> None:
    check_device_buffers(routing_case("random", 100, 8), 8, 32, 16)
    check_device_buffers(routing_case("empty_middle", 777, 64), 64, 1024, 128)


def test_cuda_graph_capture_proves_no_host_sync() -> None:
    # Capture fails if the captured code waits on the GPU; replaying with new routing proves the
    # graph reads its input (reference: tests/test_routing.py:86-108).
    from sparsebench_b200.routing import route_device

    num_tokens, num_experts, ffn_dim, block_size = 4000, 32, 256, 128
    static_idx = routing_case("random", num_tokens, num_experts, seed=1).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        route_device(static_idx, num_experts, ffn_dim, block_size)
    torch.cuda.current_stream().wait_stream(side)

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = route_device(static_idx, num_experts, ffn_dim, block_size)
    for case in ["skewed", "empty_middle"]:
        new_idx = routing_case(case, num_tokens, num_experts, seed=2)
        static_idx.copy_(new_idx.cuda())
        graph.replay()
        assert_layout_equal(captured.to_topology(), L.build_topology(new_idx, num_experts, ffn_dim, block_size))


def test_out_of_range_id_raises_without_writing_out_of_bounds() -> None:
    from sparsebench_b200.routing import route_device

    expert_idx = torch.tensor([[0, 1], [2, 8], [-1, 3]], device="cuda")
    dev = route_device(expert_idx, 8, 32, 16)
    with pytest.raises(ValueError, match="outside"):
        dev.to_topology()
    assert int(dev.tokens_per_expert.sum()) == 4
    assert dev.copy_row.tolist() == [0, 16, 32, -1, -1, 48]  # reference: tests/test_routing.py:120
    check_device_buffers(expert_idx.cpu(), 8, 32, 16)
    # The large shape carries the flag through its scan kernel too.
    for num_tokens in (30000, 140000):
        big = routing_case("random", num_tokens, 64)
        big[12345, 1] = 64
        big[num_tokens - 1, 0] = -7
        check_device_buffers(big, 64, 256, 128)


BAD_INPUTS = {
    "not_2d": (lambda: torch.tensor([0, 1], device="cuda"), 8, 32, r"\[T, k\]"),
    "too_many_experts": (lambda: torch.tensor([[0, 1]], device="cuda"), 2000, 32, "num_experts"),
    "ffn_not_multiple": (lambda: torch.tensor([[0, 1]], device="cuda"), 8, 30, "multiple"),
    "float_ids": (lambda: torch.tensor([[0.0, 1.0]], device="cuda"), 8, 32, "int32"),
    "not_contiguous": (lambda: torch.zeros(4, 4, dtype=torch.int64, device="cuda")[:, ::2], 8, 32, "contiguous"),
}


@pytest.mark.parametrize("name", BAD_INPUTS)
def test_rejects_bad_input(name: str) -> None:
    make, num_experts, ffn_dim, match = BAD_INPUTS[name]
    with pytest.raises(RuntimeError, match=match):
        route_cuda(make(), num_experts, ffn_dim, 16)
