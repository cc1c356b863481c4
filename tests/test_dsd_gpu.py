"""DSD (BSR(H) @ W) against the fp32 oracle (reference: tests/test_dsd.py). One tcgen05 kernel
serves every `version` and both block sizes (64-row blocks use half of the 128-row tile)."""

import math

import pytest
import torch

from oracle import layout as L
from oracle import moe as M
from tests.cases import CASE_NAMES, as_topology, routing_case

pytestmark = pytest.mark.gpu

VERSIONS = [pytest.param(v, id=f"v{v}") for v in (1, 2, 21, 3, 31, 4, 41, 5)]
ZEROS_DEAD_ROWS = {1, 2, 21, 3, 31}
TOL = {"rtol": 1.6e-2, "atol": 1.6e-2}


def make_inputs(case: str, num_tokens: int, num_experts: int, ffn_dim: int, d_model: int, bs: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    layout = L.build_topology(routing_case(case, num_tokens, num_experts, seed), num_experts, ffn_dim, bs)
    # H ~ N(0, 1/F), W ~ N(0, 1): each output is a sum of F terms, about N(0, 1).
    blocks = (torch.randn(layout.nnz_blocks, bs, bs, generator=g) / math.sqrt(ffn_dim)).bfloat16()
    w = torch.randn(num_experts * ffn_dim, d_model, generator=g).bfloat16()
    return layout, blocks, w


def run(blocks, w, topo, version):
    from sparsebench_b200.spmm import dsd

    return dsd(blocks.cuda(), w.cuda(), topo, version=version)


def oracle(blocks, w, layout):
    return M.dsd_rows(blocks.float(), w.float(), layout)


@pytest.mark.parametrize("version", [pytest.param(1, id="v1"), pytest.param(5, id="v5")])
@pytest.mark.parametrize("case", CASE_NAMES)
@pytest.mark.parametrize("bs", [64, 128])
@pytest.mark.parametrize(("num_experts", "f_blocks"), [(8, 1), (8, 4), (64, 1), (64, 2)], ids=["E8F1", "E8F4", "E64F1", "E64F2"])
@pytest.mark.parametrize("d_model", [128, 256, 512], ids=["D128", "D256", "D512"])
def test_matches_oracle(version: int, case: str, bs: int, num_experts: int, f_blocks: int, d_model: int) -> None:
    if version == 5 and (bs != 128 or d_model % 256 != 0):
        pytest.skip("v5 rejects block size 64 and D that is not a multiple of 256")
    layout, blocks, w = make_inputs(case, 300, num_experts, f_blocks * bs, d_model, bs)
    out = run(blocks, w, as_topology(layout), version)
    torch.testing.assert_close(out.float().cpu(), oracle(blocks, w, layout), **TOL)


@pytest.mark.parametrize("version", VERSIONS)
@pytest.mark.parametrize("bs", [64, 128])
def test_single_token(version: int, bs: int) -> None:
    if version == 5 and bs != 128:
        pytest.skip("v5 rejects block size 64")
    layout, blocks, w = make_inputs("random", 1, 8, 2 * bs, 256, bs)
    out = run(blocks, w, as_topology(layout), version)
    torch.testing.assert_close(out.float().cpu(), oracle(blocks, w, layout), **TOL)


@pytest.mark.parametrize("bs", [64, 128])
@pytest.mark.parametrize("d_model", [256, 384])
def test_asymmetric_inputs(d_model: int, bs: int) -> None:
    # reference: tests/test_dsd.py:86-102. No symmetry between rows and columns or between H and W.
    layout, _, _ = make_inputs("random", 200, 8, 2 * bs, d_model, bs)
    k_total = 8 * 2 * bs
    i = torch.arange(k_total, dtype=torch.float32)[:, None]
    j = torch.arange(d_model, dtype=torch.float32)[None, :]
    w = torch.sin(0.37 * i + 1.31 * j + 0.05 * i * j / d_model).bfloat16()
    p = torch.arange(layout.nnz_blocks, dtype=torch.float32)[:, None, None]
    r = torch.arange(bs, dtype=torch.float32)[None, :, None]
    c = torch.arange(bs, dtype=torch.float32)[None, None, :]
    blocks = (torch.cos(0.7 * r - 0.23 * c + 0.11 * p + 0.01 * r * c) / 16.0).bfloat16()
    out = run(blocks, w, as_topology(layout), 4)
    torch.testing.assert_close(out.float().cpu(), oracle(blocks, w, layout), **TOL)


def test_general_bsr_layout_not_just_the_moe_one() -> None:
    # Row blocks with 0, 1 and 3 blocks, columns in arbitrary order, a dead row block in the middle.
    from sparsebench_b200.topology import Topology

    g = torch.Generator().manual_seed(5)
    row_offsets = torch.tensor([0, 3, 3, 4, 6], dtype=torch.int32)
    col_indices = torch.tensor([5, 0, 2, 7, 1, 1], dtype=torch.int32)
    blocks = (torch.randn(6, 128, 128, generator=g) / 16).bfloat16()
    w = torch.randn(8 * 128, 256, generator=g).bfloat16()
    z = torch.zeros(0, dtype=torch.int32)
    layout = L.Layout(128, 8, 1, z.numpy(), z.numpy(), torch.zeros(512, dtype=torch.int32).numpy(), z.numpy(),
                      torch.zeros(4, dtype=torch.int32).numpy(), row_offsets.numpy(), col_indices.numpy())
    topo = Topology(128, 8, 1, z, z, z, z, z, row_offsets.cuda(), col_indices.cuda())
    expected = oracle(blocks, w, layout)
    zeroed = run(blocks, w, topo, 1).float().cpu()
    torch.testing.assert_close(zeroed, expected, **TOL)
    assert torch.all(zeroed[128:256] == 0)
    kept = run(blocks, w, topo, 5).float().cpu()
    torch.testing.assert_close(torch.cat([kept[:128], kept[256:]]), torch.cat([expected[:128], expected[256:]]), **TOL)


@pytest.mark.parametrize("version", VERSIONS)
def test_worst_case_device_topology(version: int) -> None:
    # The no-sync path: route_device's worst-case buffers go straight in.
    from sparsebench_b200.routing import route_device

    bs, num_experts, ffn_dim, d_model = 128, 64, 256, 256
    idx = routing_case("zipf", 400, num_experts)
    dev = route_device(idx.cuda(), num_experts, ffn_dim, bs)
    g = torch.Generator().manual_seed(3)
    blocks = (torch.randn(dev.col_indices.numel(), bs, bs, generator=g) / 16).bfloat16()
    w = torch.randn(num_experts * ffn_dim, d_model, generator=g).bfloat16()
    out = run(blocks, w, dev, version)
    layout = L.build_topology(idx, num_experts, ffn_dim, bs)
    assert out.shape == ((dev.row_offsets.numel() - 1) * bs, d_model)
    torch.testing.assert_close(out[: layout.num_rows].float().cpu(), oracle(blocks[: layout.nnz_blocks], w, layout), **TOL)
    if version in ZEROS_DEAD_ROWS:
        assert torch.all(out[layout.num_rows:] == 0)


def test_long_k_many_tiles() -> None:
    # F = 2048: 32 K steps per tile, several tiles per CTA at D = 1024.
    layout, blocks, w = make_inputs("random", 3000, 8, 2048, 1024, 128)
    out = run(blocks, w, as_topology(layout), 5)
    torch.testing.assert_close(out.float().cpu(), oracle(blocks, w, layout), **TOL)


BAD_INPUTS = {
    "fp32_weights": (lambda b, w: (b, w.float()), "bfloat16"),
    "fp16_blocks": (lambda b, w: (b.half(), w), "bfloat16"),
    "d_not_multiple": (lambda b, w: (b, w[:, :100].contiguous()), "multiple of 128"),
    "non_contiguous": (lambda b, w: (b, w.t().contiguous().t()), "contiguous"),
    "cpu_weights": (lambda b, w: (b, w.cpu()), "CUDA"),
}


@pytest.mark.parametrize("name", BAD_INPUTS)
def test_rejects_bad_input(name: str) -> None:
    from sparsebench_b200.spmm import dsd

    layout, blocks, w = make_inputs("random", 20, 4, 128, 256, 128)
    change, match = BAD_INPUTS[name]
    b, w2 = change(blocks.cuda(), w.cuda())
    with pytest.raises(RuntimeError, match=match):
        dsd(b, w2, as_topology(layout), version=1)


def test_rejects_unsupported_block_size_and_version() -> None:
    from sparsebench_b200 import _C

    layout, blocks, w = make_inputs("random", 20, 4, 128, 256, 128)
    with pytest.raises(RuntimeError, match="unknown dsd version"):
        run(blocks, w, as_topology(layout), 99)
    layout32 = L.build_topology(routing_case("random", 20, 4), 4, 64, 32)
    topo32 = as_topology(layout32)
    blocks32 = torch.zeros(layout32.nnz_blocks, 32, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="64 or 128"):
        _C.dsd_cuda(blocks32, w.cuda(), topo32.row_offsets, topo32.col_indices, 1)


@pytest.mark.parametrize(("bs", "d_model"), [(64, 256), (128, 128), (128, 384)])
def test_v5_rejects_shapes_it_does_not_support(bs: int, d_model: int) -> None:
    layout, blocks, w = make_inputs("random", 50, 4, 2 * bs, d_model, bs)
    with pytest.raises(RuntimeError, match="dsd v5 needs block size 128 and D a multiple of 256"):
        run(blocks, w, as_topology(layout), 5)
