"""Pins the CPU oracle (oracle/) to golden vectors produced by the reference itself
(tests/golden/make_golden.py) and to the known answers in the reference's own tests."""

import numpy as np
import pytest
import torch

from oracle import layout as L
from oracle import moe as M
from tests.cases import CASE_NAMES, FIELDS, cpu_small_inputs, digest, load_golden, random_topk, routing_case


def _golden_names() -> list[str]:
    return [str(n) for n in load_golden("topology_cases.npz")["names"]]


def _regenerate(tag: str) -> torch.Tensor:
    case, t, e, _ = tag.split("-")
    return routing_case(case, int(t[1:]), int(e[1:]))


@pytest.mark.parametrize("tag", _golden_names())
def test_layout_matches_reference_golden(tag: str) -> None:
    g = load_golden("topology_cases.npz")
    num_experts, ffn_dim, bs, full = (int(v) for v in g[f"{tag}/meta"])
    if full:
        idx = g[f"{tag}/expert_idx"]
        got = L.build_topology(idx, num_experts, ffn_dim, bs)
        for f in FIELDS:
            assert getattr(got, f).dtype == np.int32
            assert np.array_equal(getattr(got, f), g[f"{tag}/{f}"]), f
    else:
        idx = _regenerate(tag).numpy()
        assert digest(idx) == str(g[f"{tag}/idx_digest"]), "workload generator drifted from the reference's"
        got = L.build_topology(idx, num_experts, ffn_dim, bs)
        assert [digest(getattr(got, f)) for f in FIELDS] == [str(d) for d in g[f"{tag}/digests"]]


@pytest.mark.parametrize("tag", [t for t in _golden_names() if t.split("-")[0] in CASE_NAMES])
def test_workload_generators_match_reference(tag: str) -> None:
    g = load_golden("topology_cases.npz")
    idx = _regenerate(tag).numpy()
    if int(g[f"{tag}/meta"][3]):
        assert np.array_equal(idx, g[f"{tag}/expert_idx"])
    else:
        assert digest(idx) == str(g[f"{tag}/idx_digest"])


def check_invariants(topo: L.Layout, expert_idx: np.ndarray) -> None:
    """The structural properties the reference checks (tests/test_topology.py:8-45)."""
    bs, num_experts = topo.block_size, topo.num_experts
    num_tokens, k = expert_idx.shape
    flat = expert_idx.reshape(-1).astype(np.int64)
    counts = topo.tokens_per_expert.astype(np.int64)
    offsets = topo.padded_offsets.astype(np.int64)
    row_token = topo.row_token.astype(np.int64)
    copy_row = topo.copy_row.astype(np.int64)
    assert np.array_equal(counts, np.bincount(flat, minlength=num_experts))
    sizes = np.diff(offsets)
    assert offsets[0] == 0 and np.all(sizes % bs == 0)
    assert np.all(sizes >= counts) and np.all(sizes - counts < bs) and np.all(sizes[counts == 0] == 0)
    assert np.unique(copy_row).size == num_tokens * k
    assert np.all(copy_row >= offsets[flat]) and np.all(copy_row < offsets[flat] + counts[flat])
    assert np.array_equal(row_token[copy_row], np.arange(num_tokens * k) // k)
    assert int((row_token < 0).sum()) == topo.num_rows - num_tokens * k
    for e in range(num_experts):
        rows = copy_row[flat == e]
        assert np.all(rows[1:] > rows[:-1])  # stable: copy order inside an expert
    rbe = topo.row_block_expert.astype(np.int64)
    starts = np.arange(topo.num_row_blocks) * bs
    assert np.all(starts >= offsets[rbe]) and np.all(starts + bs <= offsets[rbe + 1])
    assert np.all(np.diff(topo.row_offsets) == topo.ffn_blocks)
    cols = topo.col_indices.reshape(topo.num_row_blocks, topo.ffn_blocks)
    assert np.array_equal(cols, rbe[:, None] * topo.ffn_blocks + np.arange(topo.ffn_blocks))


@pytest.mark.parametrize("case", CASE_NAMES + ["permuted_zipf"])
@pytest.mark.parametrize(("num_tokens", "block_size"), [(1, 4), (7, 4), (16, 4), (300, 16), (1000, 128)])
def test_layout_invariants(case: str, num_tokens: int, block_size: int) -> None:
    idx = routing_case(case, num_tokens, 8).numpy()
    check_invariants(L.build_topology(idx, 8, 2 * block_size, block_size), idx)


def test_int32_input_matches_int64() -> None:
    idx = routing_case("random", 50, 8).numpy()
    a, b = L.build_topology(idx, 8, 32, 16), L.build_topology(idx.astype(np.int32), 8, 32, 16)
    assert all(np.array_equal(getattr(a, f), getattr(b, f)) for f in FIELDS)


@pytest.mark.parametrize(("idx", "kwargs", "error"), [
    (np.zeros((0, 2), dtype=np.int64), {}, ValueError),
    (np.zeros(4, dtype=np.int64), {}, ValueError),
    (np.zeros((4, 2), dtype=np.float32), {}, TypeError),
    (np.array([[0, 8]]), {}, ValueError),
    (np.array([[-1, 0]]), {}, ValueError),
    (np.array([[0, 1]]), {"ffn_dim": 10}, ValueError),
    (np.array([[0, 1]]), {"block_size": 0}, ValueError),
])
def test_layout_rejects_bad_input(idx, kwargs, error) -> None:
    # Same cases as the reference (tests/test_topology.py:76-91).
    args = {"num_experts": 8, "ffn_dim": 8, "block_size": 4} | kwargs
    with pytest.raises(error):
        L.build_topology(idx, **args)


def test_device_layout_known_answer_with_bad_ids() -> None:
    # Known answer from the reference's GPU test (tests/test_routing.py:111-120): the two bad copies
    # are skipped, the four good ones placed, and the error flag is raised.
    dev = L.device_layout(np.array([[0, 1], [2, 8], [-1, 3]]), 8, 32, 16)
    assert dev.error == 1
    assert int(dev.tokens_per_expert.sum()) == 4
    assert dev.copy_row.tolist() == [0, 16, 32, -1, -1, 48]


def test_device_layout_tails() -> None:
    # Worst-case buffers are marked past the real end (reference: tests/test_routing.py:73-83).
    idx = routing_case("random", 100, 8).numpy()
    dev, trimmed = L.device_layout(idx, 8, 32, 16), L.build_topology(idx, 8, 32, 16)
    rows, rbs = trimmed.num_rows, trimmed.num_row_blocks
    max_rb, max_rows, fb = L.worst_case_sizes(200, 8, 32, 16)
    assert dev.row_token.shape == (max_rows,) and dev.row_block_expert.shape == (max_rb,)
    assert dev.error == 0
    assert np.array_equal(dev.row_token[:rows], trimmed.row_token) and np.all(dev.row_token[rows:] == -1)
    assert np.array_equal(dev.row_block_expert[:rbs], trimmed.row_block_expert)
    assert np.all(dev.row_block_expert[rbs:] == -1) and np.all(dev.col_indices[rbs * fb:] == -1)
    assert np.array_equal(dev.row_offsets[: rbs + 1], trimmed.row_offsets) and np.all(dev.row_offsets[rbs:] == rbs * fb)
    assert np.array_equal(dev.copy_row, trimmed.copy_row)


def test_bsr_round_trip() -> None:
    topo = L.build_topology(routing_case("skewed", 37, 4).numpy(), 4, 8, 4)
    blocks = np.random.default_rng(0).standard_normal((topo.nnz_blocks, 4, 4))
    dense = L.bsr_to_dense(blocks, topo)
    assert np.array_equal(L.dense_to_bsr(dense, topo), blocks)
    inside = L.bsr_to_dense(np.ones_like(blocks), topo) != 0
    assert np.all(dense[~inside] == 0) and int(inside.sum()) == blocks.size


# ---- floating point ------------------------------------------------------------------------------

def test_route_known_answer() -> None:
    # reference: tests/test_reference.py:30-35
    g = load_golden("layer_small.npz")
    idx, weight = M.route(torch.from_numpy(g["route_logits"]), k=2)
    assert idx.tolist() == [[1, 2], [0, 1]] == g["route_idx"].tolist()
    assert np.array_equal(weight.numpy(), g["route_weight"])
    assert torch.allclose(weight.sum(-1), torch.ones(2)) and torch.all(weight[:, 0] >= weight[:, 1])


def test_small_layer_matches_reference_golden() -> None:
    g = load_golden("layer_small.npz")
    _, num_experts, d_model, ffn_dim, bs = (int(v) for v in g["meta"])
    x, w1, w2, gate = (torch.from_numpy(g[k]) for k in ("x", "w1", "w2", "gate"))
    idx = torch.from_numpy(g["expert_idx"])
    tol = {"rtol": 1e-12, "atol": 1e-12}
    torch.testing.assert_close(M.moe_reference(x, idx, gate, w1, w2), torch.from_numpy(g["moe_reference"]), **tol)
    torch.testing.assert_close(M.moe_blocksparse_reference(x, idx, gate, w1, w2, bs),
                               torch.from_numpy(g["moe_blocksparse_reference"]), **tol)
    topo = L.build_topology(idx, num_experts, ffn_dim, bs)
    torch.testing.assert_close(M.group_tokens(x, topo), torch.from_numpy(g["grouped"]), rtol=0, atol=0)
    torch.testing.assert_close(M.sdd_blocks(x, w1, topo, gelu=False), torch.from_numpy(g["sdd_blocks"]), **tol)
    h = torch.nn.functional.gelu(torch.from_numpy(g["sdd_blocks"]))
    y_rows = M.dsd_rows(h, w2.reshape(num_experts * ffn_dim, d_model), topo)
    torch.testing.assert_close(y_rows, torch.from_numpy(g["dsd_rows"]), **tol)
    torch.testing.assert_close(M.ungroup_combine(y_rows, gate, topo), torch.from_numpy(g["ungroup_combine"]), **tol)


def test_cpu_small_config_matches_reference_golden() -> None:
    g = load_golden("layer_cpu_small.npz")
    x, w1, w2, logits = cpu_small_inputs()
    assert [digest(t.numpy()) for t in (x, w1, w2, logits)] == [str(d) for d in g["input_digests"]], \
        "seeded inputs differ from the ones the golden output was computed on"
    idx, gate = M.route(logits, 2)
    assert np.array_equal(idx.numpy(), g["expert_idx"]) and np.array_equal(gate.numpy(), g["gate"])
    out = M.moe_reference(x, idx, gate, w1, w2)
    torch.testing.assert_close(out[::16], torch.from_numpy(g["out_rows"]), rtol=1e-5, atol=1e-5)
    assert abs(out.double().sum().item() - float(g["out_sum"])) < 1e-2
    assert abs(out.double().abs().sum().item() - float(g["out_abs_sum"])) < 1e-1
    streamed = M.moe_reference_streamed(x, idx, gate, w1, w2)
    torch.testing.assert_close(streamed, out, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("case", CASE_NAMES)
@pytest.mark.parametrize(("num_tokens", "block_size"), [(1, 4), (29, 4), (200, 16), (300, 64)])
def test_blocksparse_matches_loop(case: str, num_tokens: int, block_size: int) -> None:
    # reference: tests/test_reference.py:50-63
    g = torch.Generator().manual_seed(0)
    num_experts, d_model, ffn_dim = 8, 24, 2 * block_size
    idx = routing_case(case, num_tokens, num_experts)
    x = torch.randn(num_tokens, d_model, dtype=torch.float64, generator=g)
    gate = torch.rand(num_tokens, 2, dtype=torch.float64, generator=g)
    w1 = torch.randn(num_experts, d_model, ffn_dim, dtype=torch.float64, generator=g) / d_model**0.5
    w2 = torch.randn(num_experts, ffn_dim, d_model, dtype=torch.float64, generator=g) / ffn_dim**0.5
    torch.testing.assert_close(M.moe_blocksparse_reference(x, idx, gate, w1, w2, block_size),
                               M.moe_reference(x, idx, gate, w1, w2), rtol=1e-10, atol=1e-10)


def test_moe_reference_rejects_mismatched_shapes() -> None:
    # reference: tests/test_reference.py:78-88
    w1, w2 = torch.zeros(4, 8, 16, dtype=torch.float64), torch.zeros(4, 16, 8, dtype=torch.float64)
    x, idx, gate = torch.zeros(5, 8, dtype=torch.float64), torch.tensor([[0, 1]]).repeat(5, 1), torch.ones(5, 2, dtype=torch.float64)
    with pytest.raises(ValueError, match="w2"):
        M.moe_reference(x, idx, gate, w1, w2.transpose(1, 2))
    with pytest.raises(ValueError, match="expert_weight"):
        M.moe_reference(x, idx, gate[:, :1], w1, w2)
    with pytest.raises(ValueError, match="x must be"):
        M.moe_reference(x[None], idx, gate, w1, w2)
