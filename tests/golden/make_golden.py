"""Generates the golden fixtures in this folder by RUNNING THE REFERENCE ITSELF.

Run once on a machine that has a checkout of the SparseBench tree; the fixtures are committed, the
reference is not and does not travel. Nothing else in the repository imports the reference.

    python tests/golden/make_golden.py <path to the SparseBench checkout>
    (or SPARSEBENCH_REFERENCE=<path> python tests/golden/make_golden.py)

Writes
  topology_cases.npz   expert_idx and every Topology field of topology.build_topology for small
                       routing cases (all five routing patterns, k in {1,2,4}, several block sizes);
                       plus SHA-256 digests of the fields for large cases.
  layer_small.npz      a tiny fp64 layer: inputs, reference.moe_reference,
                       moe_blocksparse_reference, sdd_reference / dsd_reference blocks and
                       reference.route() on fixed logits.
  layer_cpu_small.npz  the benchmark's CPU-sized configuration (seed 0, T=512 D=256 F=1024 E=8,
                       fp32): routing, gates, digests of the inputs, every 16th output row of
                       reference.moe_reference and float64 checksums of the whole output.
  rounding.npz         token_rounding.token_rounding on small score matrices (random softmax scores, and
                       rows that are permutations of a few values so that columns are full of ties):
                       scores, and the flat (token, expert, weight) list it returns.
"""

from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np
import torch

REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SPARSEBENCH_REFERENCE")
if not REFERENCE or not os.path.isdir(os.path.join(REFERENCE, "sparsebench")):
    raise SystemExit("usage: make_golden.py <path to the SparseBench checkout> (or set SPARSEBENCH_REFERENCE)")
sys.path.insert(0, REFERENCE)

from sparsebench import reference as ref  # noqa: E402
from sparsebench import token_rounding as ref_rounding  # noqa: E402
from sparsebench import topology as ref_topology  # noqa: E402
from sparsebench import workloads as ref_workloads  # noqa: E402

HERE = Path(__file__).resolve().parent
FIELDS = ("tokens_per_expert", "padded_offsets", "row_token", "copy_row", "row_block_expert", "row_offsets",
          "col_indices")


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def random_topk(num_tokens: int, num_experts: int, k: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.rand(num_tokens, num_experts, generator=g).topk(k, dim=-1).indices


def topology_cases() -> None:
    out: dict[str, np.ndarray] = {}
    names: list[str] = []

    def add(tag: str, idx: torch.Tensor, num_experts: int, ffn_dim: int, bs: int, full: bool) -> None:
        topo = ref_topology.build_topology(idx, num_experts, ffn_dim, bs)
        names.append(tag)
        out[f"{tag}/meta"] = np.array([num_experts, ffn_dim, bs, int(full)], dtype=np.int64)
        if full:
            out[f"{tag}/expert_idx"] = idx.numpy()
            for f in FIELDS:
                out[f"{tag}/{f}"] = getattr(topo, f).numpy()
        else:
            out[f"{tag}/digests"] = np.array([digest(getattr(topo, f).numpy()) for f in FIELDS])
            out[f"{tag}/idx_digest"] = np.array(digest(idx.numpy()))

    for case in ref_workloads.CASE_NAMES:
        for num_tokens, num_experts, bs in [(1, 2, 4), (13, 8, 4), (129, 8, 16), (129, 64, 128), (300, 8, 128)]:
            add(f"{case}-T{num_tokens}-E{num_experts}-bs{bs}", ref_workloads.routing_case(case, num_tokens, num_experts),
                num_experts, 2 * bs, bs, full=True)
        # Generator-reproducible large cases: digests only. (case, T, E, seed 0) -> same expert_idx.
        for num_tokens, num_experts, bs in [(1000, 256, 16), (4096, 64, 128), (20000, 1024, 128)]:
            add(f"{case}-T{num_tokens}-E{num_experts}-bs{bs}", ref_workloads.routing_case(case, num_tokens, num_experts),
                num_experts, 2 * bs, bs, full=False)
    for k in (1, 2, 4):
        for num_tokens in (1, 77):
            add(f"topk-k{k}-T{num_tokens}", random_topk(num_tokens, 16, k), 16, 32, 16, full=True)
    # No padding at all: 8 tokens x 2 copies over 2 experts = 2 blocks of 4 each.
    add("exact-multiple", torch.tensor([[0, 1]]).repeat(8, 1), 4, 8, 4, full=True)
    out["names"] = np.array(names)
    np.savez_compressed(HERE / "topology_cases.npz", **out)


def layer_small() -> None:
    g = torch.Generator().manual_seed(7)
    num_tokens, num_experts, d_model, ffn_dim, bs = 40, 4, 32, 64, 16
    x = torch.randn(num_tokens, d_model, generator=g, dtype=torch.float64)
    w1 = torch.randn(num_experts, d_model, ffn_dim, generator=g, dtype=torch.float64) / d_model**0.5
    w2 = torch.randn(num_experts, ffn_dim, d_model, generator=g, dtype=torch.float64) / ffn_dim**0.5
    idx = ref_workloads.routing_case("zipf", num_tokens, num_experts, seed=7)
    gate = torch.rand(num_tokens, 2, generator=g, dtype=torch.float64)
    topo = ref_topology.build_topology(idx, num_experts, ffn_dim, bs)
    w1_cat = w1.permute(1, 0, 2).reshape(d_model, num_experts * ffn_dim)
    w2_cat = w2.reshape(num_experts * ffn_dim, d_model)
    grouped = ref.group_tokens(x, topo)
    h = ref.sdd_reference(grouped, w1_cat, topo)
    y_rows = ref.dsd_reference(torch.nn.functional.gelu(h), w2_cat, topo)
    fixed_logits = torch.tensor([[0.1, 3.0, 2.0, -1.0], [5.0, 4.0, 0.0, 0.0]])
    route_idx, route_w = ref.route(fixed_logits, k=2)
    np.savez_compressed(
        HERE / "layer_small.npz",
        meta=np.array([num_tokens, num_experts, d_model, ffn_dim, bs], dtype=np.int64),
        x=x.numpy(), w1=w1.numpy(), w2=w2.numpy(), expert_idx=idx.numpy(), gate=gate.numpy(),
        moe_reference=ref.moe_reference(x, idx, gate, w1, w2).numpy(),
        moe_blocksparse_reference=ref.moe_blocksparse_reference(x, idx, gate, w1, w2, bs).numpy(),
        grouped=grouped.numpy(), sdd_blocks=h.numpy(), dsd_rows=y_rows.numpy(),
        ungroup_combine=ref.ungroup_combine(y_rows, gate, topo).numpy(),
        route_logits=fixed_logits.numpy(), route_idx=route_idx.numpy(), route_weight=route_w.numpy(),
    )


def layer_cpu_small() -> None:
    # Seed 0, draw order x, w1, w2, router logits; fp32 throughout.
    g = torch.Generator().manual_seed(0)
    num_tokens, d_model, ffn_dim, num_experts = 512, 256, 1024, 8
    x = torch.randn(num_tokens, d_model, generator=g)
    w1 = torch.randn(num_experts, d_model, ffn_dim, generator=g) / d_model**0.5
    w2 = torch.randn(num_experts, ffn_dim, d_model, generator=g) / ffn_dim**0.5
    logits = torch.randn(num_tokens, num_experts, generator=g)
    idx, gate = ref.route(logits, 2)
    out = ref.moe_reference(x, idx, gate, w1, w2)
    out_bs = ref.moe_blocksparse_reference(x, idx, gate, w1, w2, 128)
    np.savez_compressed(
        HERE / "layer_cpu_small.npz",
        meta=np.array([num_tokens, d_model, ffn_dim, num_experts], dtype=np.int64),
        expert_idx=idx.numpy(), gate=gate.numpy(),
        input_digests=np.array([digest(t.numpy()) for t in (x, w1, w2, logits)]),
        out_rows=out[::16].numpy(),
        out_sum=np.array(out.double().sum().item()), out_abs_sum=np.array(out.double().abs().sum().item()),
        blocksparse_max_abs_diff=np.array((out - out_bs).abs().max().item()),
        torch_version=np.array(torch.__version__),
    )


def rounding() -> None:
    out: dict[str, np.ndarray] = {}
    names = []
    cases = [("softmax", 512, 8, 2, 128, 0), ("softmax", 300, 16, 2, 32, 1), ("softmax", 1000, 64, 4, 16, 2),
             ("softmax", 77, 4, 1, 8, 4), ("softmax", 130, 8, 2, 128, 5), ("ties", 600, 8, 2, 32, 6),
             ("ties", 257, 16, 4, 16, 7)]
    for kind, num_tokens, num_experts, k, tile, seed in cases:
        g = torch.Generator().manual_seed(seed)
        if kind == "softmax":
            scores = torch.softmax(torch.randn(num_tokens, num_experts, generator=g), dim=-1)
        else:  # every row a permutation of the same E distinct values: no ties inside a row, many down a column
            values = torch.arange(1, num_experts + 1, dtype=torch.float32) / (num_experts * (num_experts + 1) / 2)
            scores = torch.stack([values[torch.randperm(num_experts, generator=g)] for _ in range(num_tokens)])
        result = ref_rounding.token_rounding(scores.clone(), k, tile)
        tag = f"{kind}-T{num_tokens}-E{num_experts}-k{k}-tile{tile}"
        names.append(tag)
        out[f"{tag}/meta"] = np.array([k, tile], dtype=np.int64)
        out[f"{tag}/scores"] = scores.numpy()
        out[f"{tag}/token"] = result.token.numpy()
        out[f"{tag}/expert"] = result.expert.numpy()
        out[f"{tag}/weight"] = result.weight.numpy()
    out["names"] = np.array(names)
    np.savez_compressed(HERE / "rounding.npz", **out)


if __name__ == "__main__":
    rounding()
    topology_cases()
    layer_small()
    layer_cpu_small()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")
