"""Seeded synthetic inputs: routing patterns and the benchmark's layer configurations.

Routing patterns follow the reference's generators (sparsebench/workloads.py:12-36) draw for draw,
so a (name, T, E, seed) triple means the same expert_idx here and there. Everything is generated on
the CPU with a seeded torch.Generator (reproducible across devices) and moved afterwards.
The reference measures on no public dataset: all of its inputs are synthetic too.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

ZIPF_EXPONENT = 1.2
CASE_NAMES = ["random", "skewed", "two_experts_only", "empty_middle", "zipf"]


def _zipf_weights(num_experts: int) -> torch.Tensor:
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float64)
    return 1.0 / ranks**ZIPF_EXPONENT


def routing_case(name: str, num_tokens: int, num_experts: int, seed: int = 0,
                 perm_seed: int | None = None) -> torch.Tensor:
    """expert_idx [T, 2] int64 on the CPU, two different experts per token.

    random            two distinct experts uniformly
    skewed            first choice always expert 0, second spread over the rest
    two_experts_only  every token picks experts 0 and 1
    empty_middle      only experts 0 and E-1 are used (in a seeded order)
    zipf              expert popularity ~ 1 / rank^1.2, two distinct draws per token
    permuted_zipf     zipf over a seeded random permutation of the experts; `perm_seed` (default:
                      `seed`) seeds the permutation alone, so that ranks with different tokens can
                      share one popularity order
    """
    g = torch.Generator().manual_seed(seed)
    if name == "random":
        return torch.rand(num_tokens, num_experts, generator=g).topk(2, dim=-1).indices
    if name == "skewed":
        second = torch.randint(1, num_experts, (num_tokens,), generator=g)
        return torch.stack([torch.zeros_like(second), second], dim=1)
    if name == "two_experts_only":
        return torch.tensor([[0, 1]]).repeat(num_tokens, 1)
    if name == "empty_middle":
        pair = torch.tensor([[0, num_experts - 1]]).repeat(num_tokens, 1)
        return pair[:, torch.randperm(2, generator=g)]
    if name == "zipf":
        return torch.multinomial(_zipf_weights(num_experts).expand(num_tokens, -1), 2, replacement=False, generator=g)
    if name == "permuted_zipf":
        if perm_seed is None:
            perm = torch.randperm(num_experts, generator=g)
        else:
            perm = torch.randperm(num_experts, generator=torch.Generator().manual_seed(perm_seed))
        picks = torch.multinomial(_zipf_weights(num_experts).expand(num_tokens, -1), 2, replacement=False, generator=g)
        return perm[picks]
    raise ValueError(name)


@dataclass(frozen=True)
class LayerConfig:
    """One synthetic MoE layer problem (top-2, block size 128)."""

    name: str
    num_tokens: int
    d_model: int
    ffn_dim: int
    num_experts: int
    routing: str
    k: int = 2

    @property
    def useful_flops(self) -> int:
        """Two matmuls over the T*k real copies; padding rows are waste, not work
        (the reference's convention, bench/bench_moe.py:235)."""
        return 4 * self.num_tokens * self.k * self.d_model * self.ffn_dim


CONFIGS = {
    # The reference's CPU-runnable case (fp32 there; bf16-rounded values here).
    "cpu_small": LayerConfig("cpu_small", 512, 256, 1024, 8, "router"),
    # Headline: fine-grained experts, uniform routing.
    "fine_grained": LayerConfig("fine_grained", 4096, 1024, 4096, 64, "random"),
    "fine_grained_zipf": LayerConfig("fine_grained_zipf", 4096, 1024, 4096, 64, "permuted_zipf"),
    "mixtral_like": LayerConfig("mixtral_like", 4096, 4096, 14336, 8, "random"),
    # Expert-parallel shape: E experts in total, T tokens per GPU.
    "expert_parallel": LayerConfig("expert_parallel", 4096, 2048, 2048, 128, "permuted_zipf"),
}


@dataclass
class LayerInputs:
    x: torch.Tensor  # [T, D]
    expert_idx: torch.Tensor  # [T, k] int64
    expert_weight: torch.Tensor  # [T, k]
    w1: torch.Tensor  # [E, D, F]
    w2: torch.Tensor  # [E, F, D]

    def to(self, device: torch.device | str) -> "LayerInputs":
        return LayerInputs(*(t.to(device) for t in (self.x, self.expert_idx, self.expert_weight, self.w1, self.w2)))


def _weights(which: int, experts: range, rows: int, cols: int, seed: int, dtype: torch.dtype) -> torch.Tensor:
    """[len(experts), rows, cols] ~ N(0, 1/rows). Every expert has its own generator, seeded by
    (seed, expert, which), so a rank can generate just its slice and still agree with the others."""
    out = torch.empty(len(experts), rows, cols, dtype=dtype)
    scale = rows**-0.5
    for slot, e in enumerate(experts):
        g = torch.Generator().manual_seed(seed * 1_000_003 + 2 * e + which)
        out[slot] = (torch.randn(rows, cols, generator=g) * scale).to(dtype)
    return out


def make_layer(cfg: LayerConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
               token_seed: int | None = None, experts: range | None = None) -> LayerInputs:
    """CPU tensors for `cfg`: x ~ N(0,1), w1 ~ N(0,1/D), w2 ~ N(0,1/F) in `dtype`; expert choice by
    cfg.routing; gates = softmax of N(0,1) logits over the selected pair ("router": logits [T, E]
    ~ N(0,1), top-2 and softmax over the picks). `token_seed` (default = seed) seeds x, routing
    and gates separately from the weights, for per-rank tokens over shared weights (the Zipf
    permutation stays seeded by `seed`). `experts` restricts w1/w2 to a slice of the experts
    (expert ids in expert_idx stay global)."""
    experts = range(cfg.num_experts) if experts is None else experts
    w1 = _weights(0, experts, cfg.d_model, cfg.ffn_dim, seed, dtype)
    w2 = _weights(1, experts, cfg.ffn_dim, cfg.d_model, seed, dtype)
    ts = seed if token_seed is None else token_seed
    gt = torch.Generator().manual_seed(1_000_003 + ts)
    x = torch.randn(cfg.num_tokens, cfg.d_model, generator=gt).to(dtype)
    if cfg.routing == "router":
        logits = torch.randn(cfg.num_tokens, cfg.num_experts, generator=gt)
        picked, expert_idx = torch.topk(logits, cfg.k, dim=-1)
        gate = torch.softmax(picked, dim=-1)
    else:
        expert_idx = routing_case(cfg.routing, cfg.num_tokens, cfg.num_experts, seed=ts, perm_seed=seed)
        gate = torch.softmax(torch.randn(cfg.num_tokens, cfg.k, generator=gt), dim=-1)
    return LayerInputs(x, expert_idx, gate.to(dtype), w1, w2)
