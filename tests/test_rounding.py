"""Token rounding: the CPU oracle against vectors produced by the reference itself, and the device kernels
against both (bit-exact token / expert lists, weights within float rounding), then the layer on a rounded
routing against the oracle's layer on the same assignment list."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe as M
from oracle import rounding as R

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "rounding.npz", allow_pickle=False)
TAGS = [str(n) for n in GOLDEN["names"]]


def golden_case(tag: str):
    k, tile = (int(v) for v in GOLDEN[f"{tag}/meta"])
    scores = torch.from_numpy(GOLDEN[f"{tag}/scores"])
    want = tuple(torch.from_numpy(GOLDEN[f"{tag}/{f}"]) for f in ("token", "expert", "weight"))
    return scores, k, tile, want


@pytest.mark.parametrize("tag", TAGS)
def test_oracle_matches_the_reference_vectors(tag: str) -> None:
    scores, k, tile, (token, expert, weight) = golden_case(tag)
    got_token, got_expert, got_weight = R.token_rounding(scores, k, tile)
    assert torch.equal(got_token, token) and torch.equal(got_expert, expert)
    torch.testing.assert_close(got_weight, weight, rtol=0, atol=0)


def test_round_counts_known_answers() -> None:
    # reference: tests/test_token_rounding.py (nearest multiple, ties down, capped by the token count)
    counts = torch.tensor([0, 1, 63, 64, 65, 127, 128, 129, 191, 192, 193, 1000])
    assert R.round_counts(counts, 128, 4096).tolist() == [0, 0, 0, 0, 128, 128, 128, 128, 128, 128, 256, 1024]
    assert R.round_counts(torch.tensor([500, 90]), 128, 300).tolist() == [256, 128]


@pytest.mark.gpu
@pytest.mark.parametrize("tag", TAGS)
def test_device_list_equals_the_reference_vectors(tag: str) -> None:
    from sparsebench_b200.rounding import token_rounding

    scores, k, tile, (token, expert, weight) = golden_case(tag)
    routed = token_rounding(scores.cuda(), k, tile)
    cap = scores.shape[0] * k + scores.shape[1] * (tile // 2)
    assert routed.token.numel() == cap
    got_token, got_expert, got_weight = (t.cpu() for t in routed.trimmed())
    assert torch.equal(got_token, token) and torch.equal(got_expert, expert)
    torch.testing.assert_close(got_weight, weight, rtol=1e-6, atol=1e-7)
    n = int(routed.count.item())
    assert bool((routed.expert[n:] == -1).all()) and bool((routed.weight[n:] == 0).all())


@pytest.mark.gpu
@pytest.mark.parametrize(("num_tokens", "num_experts", "k", "tile"), [(4096, 64, 2, 128), (3000, 8, 2, 128), (20000, 128, 4, 64)])
def test_device_list_equals_the_oracle_at_size(num_tokens: int, num_experts: int, k: int, tile: int) -> None:
    from sparsebench_b200.rounding import token_rounding

    g = torch.Generator().manual_seed(num_tokens)
    scores = torch.softmax(torch.randn(num_tokens, num_experts, generator=g), dim=-1)
    token, expert, weight = R.token_rounding(scores, k, tile)
    got_token, got_expert, got_weight = (t.cpu() for t in token_rounding(scores.cuda(), k, tile).trimmed())
    assert torch.equal(got_token, token) and torch.equal(got_expert, expert)
    torch.testing.assert_close(got_weight, weight, rtol=1e-6, atol=1e-7)
    counts = torch.bincount(got_expert, minlength=num_experts)
    assert bool((counts % tile == 0).all()), "every expert's count must be a multiple of the tile"


@pytest.mark.gpu
def test_layer_on_a_rounded_routing_without_host_sync() -> None:
    # scores -> rounding -> routing -> SDD -> DSD -> combine in one CUDA graph, replayed with new scores.
    from sparsebench_b200.rounding import moe_forward_rounded

    g = torch.Generator().manual_seed(8)
    num_tokens, num_experts, d_model, ffn_dim = 1024, 8, 256, 512
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16()
    scores = torch.softmax(torch.randn(num_tokens, num_experts, generator=g), dim=-1).cuda()
    dev = (x.cuda(), scores, w1.cuda(), w2.cuda())
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        moe_forward_rounded(*dev)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = moe_forward_rounded(*dev)
    new_scores = torch.softmax(torch.randn(num_tokens, num_experts, generator=g), dim=-1)
    scores.copy_(new_scores.cuda())
    graph.replay()
    torch.cuda.synchronize()
    token, expert, weight = R.token_rounding(new_scores, 2, 128)
    want = M.moe_assigned_reference(x.float(), token, expert, weight, w1.float(), w2.float())
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)
    from sparsebench_b200 import _C

    _C.device_status(torch.device("cuda", torch.cuda.current_device()))  # stays clean (checked by the fixture)
