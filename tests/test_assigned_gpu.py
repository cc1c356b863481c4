"""moe_forward_assigned: the layer on a flat (token, expert, weight) list
(reference: sparsebench/moe.py:59-91, tests/test_token_rounding.py:109-148)."""

import pytest
import torch

from oracle import moe as M

pytestmark = pytest.mark.gpu

TOL = {"rtol": 2e-2, "atol": 2e-2}


def make_layer(num_tokens: int, num_experts: int, d_model: int = 256, ffn_dim: int = 256, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16()
    return x, w1, w2


def run(x, token, expert, weight, w1, w2):
    from sparsebench_b200.moe import moe_forward_assigned

    return moe_forward_assigned(x.cuda(), token.cuda(), expert.cuda(), weight.cuda(), w1.cuda(), w2.cuda())


def expected(x, token, expert, weight, w1, w2):
    return M.moe_assigned_reference(x.float(), token, expert, weight.float(), w1.float(), w2.float())


@pytest.mark.parametrize("index_dtype", [torch.int64, torch.int32])
def test_any_number_of_copies_per_token(index_dtype) -> None:
    # 0 to 4 distinct experts per token, as a router that rounds per-expert counts produces.
    g = torch.Generator().manual_seed(3)
    num_tokens, num_experts = 2048, 16
    x, w1, w2 = make_layer(num_tokens, num_experts)
    copies = torch.randint(0, 5, (num_tokens,), generator=g)
    picks = torch.rand(num_tokens, num_experts, generator=g).topk(4, dim=1).indices
    keep = torch.arange(4)[None, :] < copies[:, None]
    token = torch.arange(num_tokens)[:, None].expand(-1, 4)[keep]
    expert = picks[keep]
    weight = torch.rand(token.numel(), generator=g)
    out = run(x, token.to(index_dtype), expert.to(index_dtype), weight, w1, w2)
    torch.testing.assert_close(out.float().cpu(), expected(x, token, expert, weight, w1, w2), **TOL)
    assert torch.all(out.cpu()[copies == 0] == 0)


def test_handles_0_and_3_experts_per_token() -> None:
    # reference: tests/test_token_rounding.py:121-133. Token 0: none. Token 1: one. Token 2: three.
    x, w1, w2 = make_layer(6, 4)
    token = torch.tensor([1, 2, 2, 2, 3, 3, 4, 4, 5, 5])
    expert = torch.tensor([0, 1, 2, 3, 0, 1, 2, 3, 0, 3])
    weight = torch.rand(10, generator=torch.Generator().manual_seed(1))
    out = run(x, token, expert, weight, w1, w2)
    torch.testing.assert_close(out.float().cpu(), expected(x, token, expert, weight, w1, w2), **TOL)
    assert torch.all(out[0] == 0)


def test_equals_moe_forward_for_plain_top_k() -> None:
    # reference: tests/test_token_rounding.py:136-148
    from sparsebench_b200.moe import moe_forward

    num_tokens, num_experts = 1000, 8
    x, w1, w2 = make_layer(num_tokens, num_experts)
    scores = torch.softmax(torch.randn(num_tokens, num_experts, generator=torch.Generator().manual_seed(5)), dim=-1)
    top_s, top_i = scores.topk(2, dim=1)
    weight = (top_s / top_s.sum(1, keepdim=True)).bfloat16()
    token = torch.arange(num_tokens).repeat_interleave(2)
    plain = moe_forward(x.cuda(), top_i.cuda(), weight.cuda(), w1.cuda(), w2.cuda())
    got = run(x, token, top_i.reshape(-1), weight.reshape(-1), w1, w2)
    torch.testing.assert_close(got.float(), plain.float(), **TOL)


def test_no_copies_at_all_is_zero() -> None:
    x, w1, w2 = make_layer(8, 4)
    empty = torch.zeros(0, dtype=torch.int64)
    out = run(x, empty, empty, torch.zeros(0), w1, w2)
    assert out.shape == x.shape and torch.all(out == 0)


def test_graph_capture_proves_no_host_sync() -> None:
    from sparsebench_b200.moe import moe_forward_assigned

    x, w1, w2 = (t.cuda() for t in make_layer(512, 8))
    g = torch.Generator().manual_seed(9)
    token = torch.randint(0, 512, (1500,), generator=g).cuda()
    expert = torch.randint(0, 8, (1500,), generator=g).cuda()
    weight = torch.rand(1500, generator=g).cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        moe_forward_assigned(x, token, expert, weight, w1, w2)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = moe_forward_assigned(x, token, expert, weight, w1, w2)
    new_token = torch.randint(0, 512, (1500,), generator=g)
    new_expert = torch.randint(0, 8, (1500,), generator=g)
    token.copy_(new_token.cuda())
    expert.copy_(new_expert.cuda())
    graph.replay()
    torch.cuda.synchronize()
    want = expected(x.cpu(), new_token, new_expert, weight.cpu(), w1.cpu(), w2.cpu())
    torch.testing.assert_close(out.float().cpu(), want, **TOL)
