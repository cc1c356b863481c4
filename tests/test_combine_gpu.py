"""The gate-weighted combine kernel against the reference's PyTorch lines (sparsebench/moe.py:51-55)."""

import pytest
import torch

from oracle import layout as L
from tests.cases import as_topology, random_topk, routing_case

pytestmark = pytest.mark.gpu


def expected_combine(y: torch.Tensor, copy_row: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    num_tokens, k = weight.shape
    rows = y[copy_row.long()].view(num_tokens, k, -1)
    return (rows.float() * weight.float()[..., None]).sum(dim=1).to(y.dtype)


@pytest.mark.parametrize("gate_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize(("num_tokens", "d_model", "k"), [(1, 8, 1), (37, 64, 2), (300, 256, 2), (4096, 1024, 2), (129, 320, 4)])
def test_combine_is_bit_exact_for_k_up_to_2_and_close_beyond(num_tokens: int, d_model: int, k: int, gate_dtype) -> None:
    from sparsebench_b200.spmm import combine

    g = torch.Generator().manual_seed(num_tokens)
    idx = random_topk(num_tokens, 16, k)
    topo = as_topology(L.build_topology(idx, 16, 128, 128))
    y = torch.randn(topo.num_rows, d_model, generator=g).bfloat16().cuda()
    weight = torch.rand(num_tokens, k, generator=g).to(gate_dtype).cuda()
    out = combine(y, weight, topo)
    expected = expected_combine(y, topo.copy_row, weight)
    assert out.dtype == torch.bfloat16 and out.shape == (num_tokens, d_model)
    if k <= 2:
        assert torch.equal(out, expected)  # same fp32 products, same order, one rounding
    else:
        torch.testing.assert_close(out.float(), expected.float(), rtol=1e-2, atol=1e-2)


def test_skipped_copy_contributes_zero_and_is_never_dereferenced() -> None:
    from sparsebench_b200 import _C

    y = torch.ones(4, 8, dtype=torch.bfloat16, device="cuda")
    copy_row = torch.tensor([0, -1, -1, 3], dtype=torch.int32, device="cuda")
    weight = torch.full((2, 2), 0.5, dtype=torch.bfloat16, device="cuda")
    out = _C.combine_cuda(y, copy_row, weight)
    assert torch.equal(out, torch.full((2, 8), 0.5, dtype=torch.bfloat16, device="cuda"))
