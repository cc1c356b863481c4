"""The on-device router front end (top-k + softmax over the picks) against the oracle's route()."""

import pytest
import torch

from oracle import moe as M

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(("num_tokens", "num_experts", "k"), [(2, 4, 2), (513, 8, 2), (1000, 64, 2), (300, 128, 4),
                                                              (77, 1000, 8), (64, 33, 1), (4096, 64, 2)])
def test_matches_oracle(num_tokens: int, num_experts: int, k: int, dtype) -> None:
    from sparsebench_b200 import route

    if dtype == torch.bfloat16 and num_experts > 128:
        pytest.skip("bf16 cannot hold that many distinct logits in [-4, 4]")
    g = torch.Generator().manual_seed(num_tokens + num_experts)
    # A random permutation of an evenly spaced grid per token: no two logits of a token are equal,
    # even after rounding to bf16, so the expected picks are unambiguous.
    grid = torch.linspace(-4.0, 4.0, num_experts).to(dtype)
    logits = torch.stack([grid[torch.randperm(num_experts, generator=g)] for _ in range(num_tokens)])
    idx, weight = route(logits.cuda(), k)
    want_idx, want_weight = M.route(logits, k)
    assert idx.dtype == torch.int64 and weight.dtype == dtype
    assert torch.equal(idx.cpu(), want_idx)
    tol = {"rtol": 1e-5, "atol": 1e-6} if dtype == torch.float32 else {"rtol": 2**-7, "atol": 1e-3}
    torch.testing.assert_close(weight.cpu().float(), want_weight.float(), **tol)


def test_known_answer() -> None:
    # reference: tests/test_reference.py:30-35
    from sparsebench_b200 import route

    logits = torch.tensor([[0.1, 3.0, 2.0, -1.0], [5.0, 4.0, 0.0, 0.0]], device="cuda")
    idx, weight = route(logits, k=2)
    assert idx.tolist() == [[1, 2], [0, 1]]
    assert torch.allclose(weight.sum(-1), torch.ones(2, device="cuda"))
    assert torch.all(weight[:, 0] >= weight[:, 1])


def test_nan_and_infinite_logits_follow_torch_topk() -> None:
    # torch.topk ranks NaN above every number; a row short of comparable values still yields k
    # different, valid expert ids (the routing kernel would otherwise skip the copy and raise its flag).
    from sparsebench_b200 import route

    inf, nan = float("inf"), float("nan")
    logits = torch.tensor([
        [0.5, nan, 2.0, -1.0, 1.0, 0.0, -2.0, 3.0],       # one NaN: picked first, then the maximum
        [-inf, -inf, 1.0, -inf, -inf, -inf, -inf, -inf],  # one finite value, the rest -inf
        [-inf] * 8,                                        # nothing comparable
        [nan] * 8,                                         # all NaN
        [inf, 1.0, inf, 0.0, 0.0, 0.0, 0.0, 0.0],          # two +inf: lowest id first
    ])
    idx, weight = route(logits.cuda(), 2)
    idx, weight = idx.cpu(), weight.cpu()
    want_idx, want_weight = M.route(logits, 2)
    assert idx[0].tolist() == want_idx[0].tolist() == [1, 7]
    assert idx[1].tolist()[0] == want_idx[1].tolist()[0] == 2
    assert idx[4].tolist() == [0, 2]
    for row in range(logits.shape[0]):
        picks = idx[row].tolist()
        assert len(set(picks)) == 2 and all(0 <= e < 8 for e in picks), (row, picks)
        # The picked VALUES are what torch picks (ids may differ only among equal values).
        assert torch.equal(logits[row][idx[row]].nan_to_num(nan=1e30), logits[row][want_idx[row]].nan_to_num(nan=1e30))
        assert torch.equal(weight[row].isnan(), want_weight[row].isnan()), (row, weight[row], want_weight[row])
    torch.testing.assert_close(weight[1], want_weight[1])


def test_router_to_layer_without_host_sync() -> None:
    # logits -> picks -> layer, captured in one graph and replayed with new logits.
    from sparsebench_b200 import moe_forward, route

    g = torch.Generator().manual_seed(1)
    num_tokens, num_experts, d_model, ffn_dim = 512, 8, 256, 512
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16().cuda()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16().cuda()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16().cuda()
    logits = torch.randn(num_tokens, num_experts, generator=g).cuda()

    def step():
        idx, weight = route(logits, 2)
        return moe_forward(x, idx, weight.bfloat16(), w1, w2)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    new_logits = torch.randn(num_tokens, num_experts, generator=g)
    logits.copy_(new_logits.cuda())
    graph.replay()
    torch.cuda.synchronize()
    idx, weight = M.route(new_logits, 2)
    expected = M.moe_reference(x.float().cpu(), idx, weight.bfloat16().float(), w1.float().cpu(), w2.float().cpu())
    torch.testing.assert_close(out.float().cpu(), expected, rtol=2e-2, atol=2e-2)


def test_rejects_bad_input() -> None:
    from sparsebench_b200 import route

    with pytest.raises(ValueError, match="0 < k <= E"):
        route(torch.zeros(4, 4, device="cuda"), 5)
    with pytest.raises(RuntimeError, match="k <= min"):
        route(torch.zeros(4, 16, device="cuda"), 9)


# ---- router fused into the routing kernel: logits -> layout in one launch ----------------------------------

@pytest.mark.parametrize("one_launch", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(("num_tokens", "num_experts", "k", "block_size"),
                         [(1, 4, 2, 16), (13, 8, 1, 4), (513, 8, 2, 128), (4096, 64, 2, 128), (1000, 256, 4, 128),
                          (300, 33, 8, 16), (16384, 128, 2, 128), (77, 64, 3, 128), (20000, 64, 2, 128), (64, 300, 2, 128)])
def test_route_and_layout_equals_router_then_routing(num_tokens, num_experts, k, block_size, dtype, one_launch) -> None:
    # Covers the one-launch form (k a power of two, T*k <= 32768), the shapes that fall back to two launches even
    # when it is asked for (k = 3, T*k > 32768) and the default two launches: identical results, identical to the oracle.
    import numpy as np

    from oracle import layout as L
    from sparsebench_b200 import route_and_layout

    if dtype == torch.bfloat16 and num_experts > 128:
        pytest.skip("bf16 cannot hold that many distinct logits in [-4, 4]")
    g = torch.Generator().manual_seed(num_tokens * 7 + num_experts)
    grid = torch.linspace(-4.0, 4.0, num_experts).to(dtype)
    logits = torch.stack([grid[torch.randperm(num_experts, generator=g)] for _ in range(num_tokens)])
    ffn_dim = 2 * block_size
    idx, weight, topo = route_and_layout(logits.cuda(), k, ffn_dim, block_size, one_launch)
    want_idx, want_weight = M.route(logits, k)
    assert idx.dtype == torch.int64 and weight.dtype == dtype
    assert torch.equal(idx.cpu(), want_idx)
    tol = {"rtol": 1e-5, "atol": 1e-6} if dtype == torch.float32 else {"rtol": 2**-7, "atol": 1e-3}
    torch.testing.assert_close(weight.cpu().float(), want_weight.float(), **tol)
    want = L.device_layout(want_idx, num_experts, ffn_dim, block_size)
    for field in L.Layout.FIELDS:
        assert np.array_equal(getattr(topo, field).cpu().numpy(), getattr(want, field)), field
    assert int(topo.error.item()) == 0


@pytest.mark.parametrize("one_launch", [True, False])
def test_layer_from_logits_in_a_graph_with_new_logits(one_launch: bool) -> None:
    from sparsebench_b200 import moe_forward_from_logits

    g = torch.Generator().manual_seed(3)
    num_tokens, num_experts, d_model, ffn_dim = 1024, 16, 256, 512
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16().cuda()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16().cuda()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16().cuda()
    logits = torch.randn(num_tokens, num_experts, generator=g).cuda()  # fp32: no two logits of a token are equal
    stages: list[str] = []
    moe_forward_from_logits(x, logits, w1, w2, mark=stages.append, one_launch_routing=one_launch)
    assert stages == ["routing", "SDD + GELU (fused)", "DSD", "combine"]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        moe_forward_from_logits(x, logits, w1, w2, one_launch_routing=one_launch)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = moe_forward_from_logits(x, logits, w1, w2, one_launch_routing=one_launch)
    new_logits = torch.randn(num_tokens, num_experts, generator=g)
    logits.copy_(new_logits.cuda())
    graph.replay()
    torch.cuda.synchronize()
    idx, weight = M.route(new_logits, 2)
    expected = M.moe_reference(x.float().cpu(), idx, weight.float(), w1.float().cpu(), w2.float().cpu())
    torch.testing.assert_close(out.float().cpu(), expected, rtol=2e-2, atol=2e-2)
