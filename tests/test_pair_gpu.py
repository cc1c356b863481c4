"""SDD and DSD on pairs of thread blocks (tcgen05 cta_group::2): two row blocks of one expert per tile.

The pair kernel serves layouts whose experts have several row blocks each. Checked here against the CPU
oracle (the reference's tolerance, 1.6e-2) and against the one-CTA kernel on the same inputs (same K order
and fp32 accumulation: bit-identical), on layouts with odd row-block counts (a half-idle pair), unused
experts, a single expert, padding-row skipping, and through the layer.
"""

import numpy as np
import pytest
import torch

from oracle import layout as L
from oracle import moe as M
from tests.cases import routing_case

pytestmark = pytest.mark.gpu


def _inputs(case: str, num_tokens: int, num_experts: int, d_model: int, ffn_dim: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16()
    gate = torch.rand(num_tokens, 2, generator=g).bfloat16()
    idx = routing_case(case, num_tokens, num_experts, seed=seed)
    return x, idx, gate, w1, w2


CASES = [("random", 1000, 2, 256, 512), ("skewed", 700, 4, 512, 256), ("empty_middle", 900, 4, 256, 512),
         ("two_experts_only", 130, 8, 256, 256), ("random", 2100, 3, 512, 1024)]


@pytest.mark.parametrize(("case", "num_tokens", "num_experts", "d_model", "ffn_dim"), CASES)
@pytest.mark.parametrize("skip_padding", [False, True])
def test_pair_kernels_match_oracle_and_one_cta_kernels(monkeypatch, case, num_tokens, num_experts, d_model, ffn_dim,
                                                       skip_padding) -> None:
    from sparsebench_b200 import _C
    from sparsebench_b200.routing import route_device

    x, idx, _, w1, w2 = _inputs(case, num_tokens, num_experts, d_model, ffn_dim)
    topo = route_device(idx.cuda(), num_experts, ffn_dim, 128)
    layout = L.build_topology(idx, num_experts, ffn_dim, 128)
    nnz, rows = layout.nnz_blocks, layout.num_row_blocks * 128
    args = (x.cuda(), w1.cuda(), topo.row_token, topo.row_block_expert, topo.row_offsets, topo.col_indices.numel(), True,
            skip_padding)
    monkeypatch.setenv("SB_GEMM_PAIRS", "0")
    h_one = _C.sdd_cuda(*args, topo.padded_offsets)
    monkeypatch.setenv("SB_GEMM_PAIRS", "2")
    h_pair = _C.sdd_cuda(*args, topo.padded_offsets)
    torch.cuda.synchronize()
    want_h = M.sdd_blocks(x.float(), w1.float(), layout, gelu=True)
    live = torch.from_numpy(np.repeat(layout.row_token >= 0, 1)).view(-1, 128)  # [row blocks, 128] real rows
    fb = ffn_dim // 128
    got = h_pair[:nnz].float().cpu().view(-1, fb, 128, 128)
    one = h_one[:nnz].float().cpu().view(-1, fb, 128, 128)
    want = want_h.view(-1, fb, 128, 128)
    mask = live[:, None, :, None].expand_as(got)
    if not skip_padding:
        mask = torch.ones_like(mask)
        assert torch.all(got[~live[:, None, :, None].expand_as(got)] == 0), "padding rows must come out exactly 0"
    torch.testing.assert_close(got[mask], want[mask], rtol=1.6e-2, atol=1.6e-2)
    assert torch.equal(got[mask], one[mask]), "pair kernel and one-CTA kernel disagree"

    # DSD on the oracle's H (rounded to bf16), padding rows poisoned when they are to be skipped.
    h_in = torch.zeros(topo.col_indices.numel(), 128, 128, dtype=torch.bfloat16)
    h_in[:nnz] = want_h.bfloat16()
    if skip_padding:
        poison = h_in[:nnz].view(-1, fb, 128, 128)
        # Rows in groups of 32 that are all padding: the kernel must not even load them.
        dead_row = (~live).view(-1, 4, 32).all(dim=2, keepdim=True).expand(-1, 4, 32).reshape(-1, 128)
        poison.permute(0, 2, 1, 3)[dead_row] = float("nan")
    w2_cat = w2.view(num_experts * ffn_dim, d_model).cuda()
    dsd_args = (h_in.cuda(), w2_cat, topo.row_offsets, topo.col_indices, 5, topo.row_token if skip_padding else None)
    monkeypatch.setenv("SB_GEMM_PAIRS", "0")
    y_one = _C.dsd_cuda(*dsd_args, topo.padded_offsets)
    monkeypatch.setenv("SB_GEMM_PAIRS", "2")
    y_pair = _C.dsd_cuda(*dsd_args, topo.padded_offsets)
    torch.cuda.synchronize()
    want_y = M.dsd_rows(h_in[:nnz].float().nan_to_num(0.0), w2_cat.float().cpu(), layout)
    real = torch.from_numpy(layout.row_token >= 0)
    keep = real if skip_padding else torch.ones_like(real)
    torch.testing.assert_close(y_pair[:rows].float().cpu()[keep], want_y[keep], rtol=1.6e-2, atol=1.6e-2)
    assert torch.equal(y_pair[:rows][keep.cuda()], y_one[:rows][keep.cuda()])


@pytest.mark.parametrize(("case", "num_tokens", "num_experts", "d_model", "ffn_dim"),
                         [("random", 2048, 2, 512, 1024), ("zipf", 1500, 4, 256, 768), ("random", 4096, 8, 1024, 2048)])
def test_layer_runs_on_pairs_where_experts_are_large(case, num_tokens, num_experts, d_model, ffn_dim) -> None:
    # Worst-case row blocks >= 4 per expert: moe_forward picks the pair kernels by itself.
    from sparsebench_b200 import moe_forward

    x, idx, gate, w1, w2 = _inputs(case, num_tokens, num_experts, d_model, ffn_dim, seed=4)
    assert (num_tokens * 2 + num_experts * 127) // 128 >= 4 * num_experts
    out = moe_forward(x.cuda(), idx.cuda(), gate.cuda(), w1.cuda(), w2.cuda())
    want = M.moe_reference_streamed(x, idx, gate, w1, w2)
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)
