"""Out-of-bounds write check without a memory checker: every output buffer of the four layer kernels is a window
in the middle of a larger allocation whose surroundings hold a sentinel; after the call, through the raw C ABI, the
sentinel must be intact on both sides of every window (and the window must hold the right result). Catches a kernel
that stores one row, block or element past what its contract says, which a tolerance check of the result cannot."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import layout as L
from sparsebench_b200 import _C, _lib
from tests.cases import routing_case

pytestmark = pytest.mark.gpu

GUARD = 4096  # elements of sentinel on each side of a window


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def windows(sizes: list[int], dtype: torch.dtype, sentinel: float | int):
    """One buffer: guard | window 0 | guard | window 1 | ... | guard, each window 256-byte aligned."""
    elem = torch.empty(0, dtype=dtype).element_size()
    align = 256 // elem
    padded = [(s + align - 1) // align * align for s in sizes]
    total = GUARD + sum(p + GUARD for p in padded)
    buf = torch.full((total,), sentinel, dtype=dtype, device="cuda")
    views, spans, off = [], [], GUARD
    for s, p in zip(sizes, padded):
        views.append(buf[off:off + s])
        spans.append((off, off + s))
        off += p + GUARD
    return buf, views, spans


def assert_guards_intact(buf: torch.Tensor, spans, sentinel, what: str) -> None:
    inside = torch.zeros(buf.numel(), dtype=torch.bool, device=buf.device)
    for a, b in spans:
        inside[a:b] = True
    outside = buf[~inside]
    bad = outside != sentinel if not isinstance(sentinel, float) or sentinel == sentinel else ~outside.isnan()
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements outside the output windows were overwritten"


@pytest.mark.parametrize(("case", "num_tokens", "num_experts"), [("zipf", 1000, 8), ("random", 4096, 64), ("skewed", 70_000, 16)])
def test_layer_kernels_write_only_inside_their_outputs(case: str, num_tokens: int, num_experts: int) -> None:
    lib = _lib.load()
    d_model, ffn_dim, k = 256, 512, 2
    if num_tokens > 8192:
        d_model, ffn_dim = 128, 256  # keeps the large-routing case small in bytes; SDD/DSD are skipped for it
    g = torch.Generator().manual_seed(1)
    idx = routing_case(case, num_tokens, num_experts, seed=2).cuda()
    n = num_tokens * k
    rb, rows, fb = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _lib.check(lib.sb_route_sizes(n, num_experts, ffn_dim, 128, ctypes.byref(rb), ctypes.byref(rows), ctypes.byref(fb)))
    rb, rows, fb = rb.value, rows.value, fb.value
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # ---- routing: eight int32 outputs
    sizes = [num_experts, num_experts + 1, rows, n, rb, rb + 1, rb * fb, 1]
    ibuf, outs, ispans = windows(sizes, torch.int32, -77)
    work = torch.empty(max(1, lib.sb_route_workspace_bytes(n, num_experts)), dtype=torch.uint8, device="cuda")
    _lib.check(lib.sb_route(_ptr(idx), 1, n, k, num_experts, fb, 128, rb, *map(_ptr, outs), _ptr(work), stream))
    torch.cuda.synchronize()
    assert_guards_intact(ibuf, ispans, -77, "routing")
    want = L.device_layout(idx.cpu(), num_experts, ffn_dim, 128)
    for name, got in zip(L.Layout.FIELDS, outs):
        assert np.array_equal(got.cpu().numpy(), getattr(want, name)), name
    if num_tokens > 8192:
        return
    tokens_per_expert, padded_offsets, row_token, copy_row, row_block_expert, row_offsets, col_indices, _ = outs

    # ---- SDD: blocks [rb * fb, 128, 128]; DSD: y [rb * 128, D]; combine: out [T, D]
    x = torch.randn(num_tokens, d_model, generator=g).bfloat16().cuda()
    w1 = (torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5).bfloat16().cuda()
    w2 = (torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5).bfloat16().cuda()
    gate = torch.rand(num_tokens, k, generator=g).bfloat16().cuda()
    nan = float("nan")
    fbuf, (h, y, out), fspans = windows([rb * fb * 128 * 128, rb * 128 * d_model, num_tokens * d_model], torch.bfloat16, nan)
    status = _C.device_status(torch.device("cuda", torch.cuda.current_device()))
    _lib.check(lib.sb_sdd(_ptr(x), _ptr(w1), _ptr(row_token), _ptr(row_block_expert), _ptr(row_offsets), _ptr(h),
                          num_tokens, d_model, ffn_dim, num_experts, rb, 1, 0, None, _ptr(status), stream))
    _lib.check(lib.sb_dsd(_ptr(h), rb * fb, _ptr(w2), num_experts * ffn_dim, d_model, _ptr(row_offsets), _ptr(col_indices),
                          rb, 128, 0, None, _ptr(y), None, 0, _ptr(status), stream))
    _lib.check(lib.sb_combine(_ptr(y), _ptr(copy_row), _ptr(gate), 0, _ptr(out), num_tokens, k, d_model, stream))
    torch.cuda.synchronize()
    assert_guards_intact(fbuf, fspans, nan, "sdd / dsd / combine")
    # Inside the windows: live rows are written, rows of dead row blocks are not (they keep the sentinel).
    live_rows = int(want.padded_offsets[-1])
    assert not bool(h[: live_rows // 128 * fb * 128 * 128].isnan().any())
    assert bool(h[live_rows // 128 * fb * 128 * 128:].isnan().all())
    assert not bool(y[: live_rows * d_model].isnan().any()) and bool(y[live_rows * d_model:].isnan().all())
    from sparsebench_b200 import moe_forward

    expected = moe_forward(x, idx, gate, w1, w2)
    torch.testing.assert_close(out.view(num_tokens, d_model).float(), expected.float(), rtol=0, atol=0)
