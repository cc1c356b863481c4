"""Shared helpers for the tests: golden fixtures, oracle <-> product conversions, seeded inputs."""

from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

from oracle import layout as oracle_layout
from sparsebench_b200.topology import Topology
from sparsebench_b200.workloads import CASE_NAMES, routing_case

__all__ = ["CASE_NAMES", "GOLDEN", "routing_case", "load_golden", "as_topology", "digest", "random_topk",
           "cpu_small_inputs", "assert_layout_equal"]

GOLDEN = Path(__file__).resolve().parent / "golden"
FIELDS = oracle_layout.Layout.FIELDS


def load_golden(name: str):
    return np.load(GOLDEN / name, allow_pickle=False)


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def random_topk(num_tokens: int, num_experts: int, k: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.rand(num_tokens, num_experts, generator=g).topk(k, dim=-1).indices


def as_topology(layout: oracle_layout.Layout, device: str | torch.device = "cuda") -> Topology:
    """An oracle layout as the product's Topology (int32 tensors on `device`)."""
    tensors = {f: torch.from_numpy(getattr(layout, f)).to(device) for f in FIELDS}
    return Topology(layout.block_size, layout.num_experts, layout.ffn_blocks, **tensors)


def assert_layout_equal(actual: Topology, expected: oracle_layout.Layout) -> None:
    """Bit-exact, field by field, dtype included."""
    assert (actual.block_size, actual.num_experts, actual.ffn_blocks) == (
        expected.block_size, expected.num_experts, expected.ffn_blocks)
    for f in FIELDS:
        got = getattr(actual, f)
        assert got.dtype == torch.int32, f
        assert np.array_equal(got.cpu().numpy(), getattr(expected, f)), f"{f} differs"


def cpu_small_inputs():
    """The benchmark's CPU-sized configuration: seed 0, draw order x, w1, w2, router logits, fp32."""
    g = torch.Generator().manual_seed(0)
    num_tokens, d_model, ffn_dim, num_experts = 512, 256, 1024, 8
    x = torch.randn(num_tokens, d_model, generator=g)
    w1 = torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5
    w2 = torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5
    logits = torch.randn(num_tokens, num_experts, generator=g)
    return x, w1, w2, logits
