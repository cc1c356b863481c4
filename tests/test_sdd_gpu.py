"""SDD (gather + X@W1 + GELU into BSR blocks) against the fp32 oracle (reference: tests/test_sdd.py)."""

import pytest
import torch

from oracle import layout as L
from oracle import moe as M
from tests.cases import CASE_NAMES, as_topology, routing_case

pytestmark = pytest.mark.gpu

TOL = {"rtol": 1.6e-2, "atol": 1.6e-2}  # bf16 output rounding; layout bugs are far bigger


def make_inputs(case: str, num_tokens: int, num_experts: int, d_model: int, ffn_dim: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    idx = routing_case(case, num_tokens, num_experts, seed)
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    return idx, x, w1


def run_sdd(x, w1, topo, gelu=True):
    from sparsebench_b200.spmm import sdd

    return sdd(x.cuda(), w1.cuda(), topo, gelu=gelu)


def expected(x, w1, layout, gelu):
    return M.sdd_blocks(x.float(), w1.float(), layout, gelu)


@pytest.mark.parametrize("case", CASE_NAMES)
@pytest.mark.parametrize(("num_experts", "d_model", "ffn_dim"), [(8, 128, 256), (8, 320, 512), (64, 64, 256)],
                         ids=["E8D128F256", "E8D320F512", "E64D64F256"])
def test_sdd_matches_oracle(case: str, num_experts: int, d_model: int, ffn_dim: int) -> None:
    idx, x, w1 = make_inputs(case, 300, num_experts, d_model, ffn_dim)
    layout = L.build_topology(idx, num_experts, ffn_dim, 128)
    out = run_sdd(x, w1, as_topology(layout))
    torch.testing.assert_close(out.float().cpu(), expected(x, w1, layout, True), **TOL)


def test_sdd_without_gelu() -> None:
    idx, x, w1 = make_inputs("zipf", 200, 8, 128, 256)
    layout = L.build_topology(idx, 8, 256, 128)
    out = run_sdd(x, w1, as_topology(layout), gelu=False)
    torch.testing.assert_close(out.float().cpu(), expected(x, w1, layout, False), **TOL)


@pytest.mark.parametrize(("num_tokens", "num_experts"), [(1500, 2), (1300, 3), (4100, 4)])
def test_sdd_many_row_blocks_per_expert(num_tokens: int, num_experts: int) -> None:
    # At >= 4 row blocks per expert the kernel walks its tiles in bands of 8 row blocks (row block
    # fastest, then column slice); the row-block counts here leave a short last band (24, 22, 66 + dead ones).
    idx, x, w1 = make_inputs("zipf", num_tokens, num_experts, 128, 768)
    layout = L.build_topology(idx, num_experts, 768, 128)
    out = run_sdd(x, w1, as_topology(layout))
    torch.testing.assert_close(out.float().cpu(), expected(x, w1, layout, True), **TOL)
    from sparsebench_b200.routing import route_device
    from sparsebench_b200.spmm import sdd

    topo = route_device(idx.cuda(), num_experts, 768, 128)  # worst-case sized: dead row blocks at the end
    blocks = sdd(x.cuda(), w1.cuda(), topo)
    live = int(topo.row_offsets[-1])
    assert torch.equal(blocks[:live], out[:live])


def test_sdd_single_token_is_mostly_padding() -> None:
    # 1 token, 2 copies: each row block is 1 real row + 127 zero-filled ones.
    idx, x, w1 = make_inputs("random", 1, 8, 128, 256)
    layout = L.build_topology(idx, 8, 256, 128)
    out = run_sdd(x, w1, as_topology(layout), gelu=False).float().cpu()
    torch.testing.assert_close(out, expected(x, w1, layout, False), **TOL)
    assert torch.all(out[:, 1:, :] == 0), "padding rows must come out exactly zero"


def test_sdd_asymmetric_inputs() -> None:
    # Smooth structured values with no symmetry between rows, columns and K, so that a transposed
    # operand, a swapped K sub-step or a mis-swizzled chunk cannot hide behind random data.
    num_tokens, num_experts, d_model, ffn_dim = 200, 4, 192, 512
    idx = routing_case("random", num_tokens, num_experts)
    t = torch.arange(num_tokens, dtype=torch.float32)[:, None]
    d = torch.arange(d_model, dtype=torch.float32)[None, :]
    x = torch.cos(0.7 * t - 0.23 * d + 0.01 * t * d / d_model).bfloat16()
    e = torch.arange(num_experts, dtype=torch.float32)[:, None, None]
    i = torch.arange(d_model, dtype=torch.float32)[None, :, None]
    j = torch.arange(ffn_dim, dtype=torch.float32)[None, None, :]
    w1 = (torch.sin(0.37 * i + 1.31 * j + 0.9 * e + 0.05 * i * j / ffn_dim) / d_model**0.5).bfloat16()
    layout = L.build_topology(idx, num_experts, ffn_dim, 128)
    out = run_sdd(x, w1, as_topology(layout), gelu=False)
    torch.testing.assert_close(out.float().cpu(), expected(x, w1, layout, False), **TOL)


def test_sdd_gelu_is_the_erf_form_to_bf16_rounding() -> None:
    # One-hot token rows make every pre-activation an exact copy of a weight, so the only arithmetic
    # left is the GELU itself: it must agree with the erf form (not the tanh form) to the last bf16
    # bit or one next to it, over the whole range where GELU is not trivially 0 or x.
    num_tokens, d_model, ffn_dim = 64, 64, 256
    x = torch.eye(num_tokens, d_model).bfloat16()
    w1 = torch.linspace(-7.0, 7.0, d_model * ffn_dim).reshape(1, d_model, ffn_dim).bfloat16()
    idx = torch.zeros(num_tokens, 1, dtype=torch.int64)
    layout = L.build_topology(idx, 1, ffn_dim, 128)
    out = run_sdd(x, w1, as_topology(layout)).float().cpu()
    want = torch.nn.functional.gelu(w1[0].float()).bfloat16().float()  # [64 tokens, 256]
    got = out[:, :64, :].permute(1, 0, 2).reshape(64, ffn_dim)  # blocks [2,128,128] -> rows of tokens
    torch.testing.assert_close(got, want, rtol=2**-7, atol=2e-6)
    tanh_form = torch.nn.functional.gelu(w1[0].float(), approximate="tanh")
    assert (got - want).abs().max() < (tanh_form - torch.nn.functional.gelu(w1[0].float())).abs().max()


def test_sdd_worst_case_device_topology() -> None:
    # The no-sync path: worst-case buffers straight from route_device.
    from sparsebench_b200.routing import route_device

    idx, x, w1 = make_inputs("zipf", 400, 64, 128, 256)
    dev = route_device(idx.cuda(), 64, 256, 128)
    out = run_sdd(x, w1, dev)
    layout = L.build_topology(idx, 64, 256, 128)
    assert out.shape[0] == dev.col_indices.numel()
    torch.testing.assert_close(out[: layout.nnz_blocks].float().cpu(), expected(x, w1, layout, True), **TOL)


def test_sdd_many_tiles_per_cta() -> None:
    # More tiles than SMs: every CTA walks several tiles, both TMEM accumulators and several
    # trips round the stage ring.
    idx, x, w1 = make_inputs("random", 3000, 16, 256, 1024)
    layout = L.build_topology(idx, 16, 1024, 128)
    out = run_sdd(x, w1, as_topology(layout))
    torch.testing.assert_close(out.float().cpu(), expected(x, w1, layout, True), **TOL)


BAD = {
    "fp32_x": (lambda x, w1: (x.float(), w1), "bfloat16"),
    "f_not_256": (lambda x, w1: (x, w1[:, :, :128].contiguous()), "multiple of 256"),
    "d_not_64": (lambda x, w1: (x[:, :96].contiguous(), w1[:, :96].contiguous()), "multiple of 64"),
    "d_mismatch": (lambda x, w1: (x[:, :64].contiguous(), w1), r"\[T, D\]"),
}


@pytest.mark.parametrize("name", BAD)
def test_sdd_rejects_bad_input(name: str) -> None:
    from sparsebench_b200 import _C

    idx, x, w1 = make_inputs("random", 20, 4, 128, 256)
    topo = as_topology(L.build_topology(idx, 4, 256, 128))
    change, match = BAD[name]
    xx, ww = change(x.cuda(), w1.cuda())
    with pytest.raises(RuntimeError, match=match):
        _C.sdd_cuda(xx, ww, topo.row_token, topo.row_block_expert, topo.row_offsets, topo.col_indices.numel(), True)


def test_sdd_rejects_block_size_64() -> None:
    idx, x, w1 = make_inputs("random", 20, 4, 128, 256)
    with pytest.raises(ValueError, match="block size 128"):
        run_sdd(x, w1, as_topology(L.build_topology(idx, 4, 256, 64)))
