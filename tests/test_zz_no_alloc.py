"""Routing through the entry point that needs no device allocation from its caller.

sb_route_static_scratch keeps the chunk histograms of the large launch shape in an array that is
part of the library, for callers that have no way to hand over scratch memory: a binding that can
only pass pointers along, or a process that may not call cudaMalloc once it is serving (the call
synchronises the device, which this path promises never to do). This file checks, through the C ABI,
that it leaves exactly what sb_route leaves in every output buffer, twice in a row with different
routing (the shared array still holds the first call's contents when the second one runs), that
those buffers are also what the CPU oracle of the layout says they must be, and that it refuses
sizes the array cannot hold. It is named so that pytest collects it last.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import layout as L
from sparsebench_b200 import _lib
from tests.cases import routing_case

pytestmark = pytest.mark.gpu

NAMES = ("tokens_per_expert", "padded_offsets", "row_token", "copy_row", "row_block_expert", "row_offsets",
         "col_indices", "error")


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _route(lib, expert_idx: torch.Tensor, num_experts: int, ffn_dim: int, block_size: int, static: bool):
    """Calls sb_route (with a workspace of ours) or sb_route_static_scratch (without) on the same
    freshly poisoned output buffers and returns them."""
    n, k = expert_idx.numel(), expert_idx.shape[1]
    rb, rows, fb = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _lib.check(lib.sb_route_sizes(n, num_experts, ffn_dim, block_size, ctypes.byref(rb), ctypes.byref(rows),
                                  ctypes.byref(fb)))
    sizes = [num_experts, num_experts + 1, rows.value, n, rb.value, rb.value + 1, rb.value * fb.value, 1]
    outs = [torch.full((s,), -77, dtype=torch.int32, device="cuda") for s in sizes]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = (_ptr(expert_idx), int(expert_idx.dtype == torch.int64), n, k, num_experts, fb.value, block_size, rb.value)
    if static:
        _lib.check(lib.sb_route_static_scratch(*head, *map(_ptr, outs), stream))
    else:
        work = torch.empty(max(1, lib.sb_route_workspace_bytes(n, num_experts)), dtype=torch.uint8, device="cuda")
        _lib.check(lib.sb_route(*head, *map(_ptr, outs), _ptr(work), stream))
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in outs]


@pytest.mark.parametrize(("num_tokens", "num_experts"), [(150_000, 64), (140_000, 512), (4096, 64)],
                         ids=["300k-copies-E64", "280k-copies-E512", "one-launch-shape"])
def test_same_buffers_as_sb_route_two_calls_in_a_row(num_tokens: int, num_experts: int) -> None:
    lib = _lib.load()
    for call, (case, seed) in enumerate([("skewed", 1), ("random", 2)]):
        idx = routing_case(case, num_tokens, num_experts, seed=seed).cuda()
        if call == 1:
            idx[num_tokens // 2, 1] = num_experts  # one bad id: the error word travels through the scratch too
        expected = _route(lib, idx, num_experts, 256, 128, static=False)
        got = _route(lib, idx, num_experts, 256, 128, static=True)
        for name, a, b in zip(NAMES, got, expected):
            assert np.array_equal(a, b), f"call {call}: {name} differs from sb_route"
        assert int(got[-1][0]) == call
        # And against the CPU oracle directly, so that this file stands by itself.
        want = L.device_layout(idx.cpu(), num_experts, 256, 128)
        for name, a in zip(NAMES[:-1], got):
            assert np.array_equal(a, getattr(want, name)), f"call {call}: {name} differs from the oracle"
        assert int(got[-1][0]) == want.error


def test_rejects_what_the_array_cannot_hold() -> None:
    lib = _lib.load()
    n, num_experts = 4_000_000, 1024  # needs 8 MB of chunk histograms; the array is 1 MiB
    assert lib.sb_route_workspace_bytes(n, num_experts) > 1 << 20
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes before any launch
    rc = lib.sb_route_static_scratch(one, 1, n, 2, num_experts, 2, 128, (n + num_experts * 127) // 128,
                                     one, one, one, one, one, one, one, one, None)
    assert rc == 1
    text = lib.sb_last_error().decode()
    assert "static scratch" in text and "1048576" in text and "sb_route" in text
