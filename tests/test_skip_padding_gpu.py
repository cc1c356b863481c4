"""skip_padding_rows: SDD does not store, and DSD neither loads nor stores, groups of 32 rows that are
all padding. Every other row must come out bit-identical to the plain kernels, and DSD must not even
look at the skipped rows of H (they are poisoned with NaN here)."""

import pytest
import torch

from tests.cases import routing_case

pytestmark = pytest.mark.gpu

SHAPES = [
    # T, D, F, E, routing
    (64, 256, 256, 4, "random"),
    (300, 256, 512, 8, "zipf"),
    (1000, 512, 1024, 16, "skewed"),
    (2048, 384, 768, 32, "empty_middle"),  # D % 256 != 0: the 128-wide DSD instance
    (4096, 1024, 4096, 64, "random"),
    (4096, 1024, 4096, 64, "zipf"),
]


def make_layer(num_tokens: int, num_experts: int, d_model: int, ffn_dim: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16()
    return x, w1, w2


def live_group_rows(topo) -> torch.Tensor:
    """[num_row_blocks * bs] bool: the row belongs to a group of 32 that holds at least one real row."""
    bs = topo.block_size
    first = topo.row_token.view(-1, bs // 32, 32)[:, :, 0] >= 0
    # padding sits at the end of each row block, so a group is live iff its first row is
    any_live = (topo.row_token.view(-1, bs // 32, 32) >= 0).any(dim=2)
    assert torch.equal(first, any_live)
    return first.repeat_interleave(32, dim=1).reshape(-1)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "-".join(map(str, s)))
def test_sdd_and_dsd_skip_padding_rows(shape) -> None:
    from sparsebench_b200.routing import route_device
    from sparsebench_b200.spmm import dsd, sdd

    T, D, F, E, case = shape
    x, w1, w2 = (t.cuda() for t in make_layer(T, E, D, F))
    topo = route_device(routing_case(case, T, E).cuda(), E, F, 128)
    w2_cat = w2.view(E * F, D)
    version = 5 if D % 256 == 0 else 4
    h_ref = sdd(x, w1, topo, gelu=True)
    y_ref = dsd(h_ref, w2_cat, topo, version=version)

    rows = live_group_rows(topo)                      # per layout row
    live_blocks = int(topo.row_offsets[-1])
    blocks_per_rb = F // 128
    block_rows = rows.view(-1, 1, 128).expand(-1, blocks_per_rb, 128).reshape(-1, 128)  # [nnz, 128] in BSR order
    num_rb_live = live_blocks // blocks_per_rb

    # SDD: every row of a live group equals the plain kernel's. Layout row blocks are live in order
    # (dead ones last), so the first live_blocks blocks are rows' first num_rb_live row blocks.
    live_rb = (topo.row_offsets[1:] > topo.row_offsets[:-1]).cpu()
    assert bool(live_rb[:num_rb_live].all()) and not bool(live_rb[num_rb_live:].any())
    h = sdd(x, w1, topo, gelu=True, skip_padding_rows=True)
    mask = block_rows[:live_blocks]
    assert torch.equal(h[:live_blocks][mask], h_ref[:live_blocks][mask])

    # DSD on poisoned input: NaN wherever a skipped group sits. Rows of live groups must not change.
    poisoned = h_ref.clone()
    poisoned[:live_blocks][~mask] = float("nan")
    y = dsd(poisoned, w2_cat, topo, version=version, skip_padding_rows=True)
    torch.cuda.synchronize()
    live_rows = rows & live_rb.cuda().repeat_interleave(128)
    assert not torch.isnan(y[live_rows].float()).any()
    assert torch.equal(y[live_rows], y_ref[live_rows])
    # ... and the two chained, as the layer runs them.
    y2 = dsd(h, w2_cat, topo, version=version, skip_padding_rows=True)
    assert torch.equal(y2[live_rows], y_ref[live_rows])


def test_dsd_skip_padding_rows_block_size_64() -> None:
    from sparsebench_b200.routing import route_device
    from sparsebench_b200.spmm import dsd

    T, D, F, E = 700, 256, 512, 8
    _, _, w2 = (t.cuda() for t in make_layer(T, E, D, F))
    topo = route_device(routing_case("zipf", T, E).cuda(), E, F, 64)
    nnz = topo.col_indices.numel()
    g = torch.Generator().manual_seed(3)
    blocks = torch.randn(nnz, 64, 64, generator=g).bfloat16().cuda()
    y_ref = dsd(blocks, w2.view(E * F, D), topo, version=4)
    rows = live_group_rows(topo)
    live_rb = topo.row_offsets[1:] > topo.row_offsets[:-1]
    live_rows = rows & live_rb.repeat_interleave(64)
    live_blocks = int(topo.row_offsets[-1])
    block_rows = rows.view(-1, 1, 64).expand(-1, F // 64, 64).reshape(-1, 64)[:live_blocks]
    poisoned = blocks.clone()
    poisoned[:live_blocks][~block_rows] = float("nan")
    y = dsd(poisoned, w2.view(E * F, D), topo, version=4, skip_padding_rows=True)
    assert not torch.isnan(y[live_rows].float()).any()
    assert torch.equal(y[live_rows], y_ref[live_rows])
