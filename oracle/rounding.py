"""Token rounding, CPU restatement. TEST INFRASTRUCTURE (see oracle/__init__.py).

Restates the reference's sparsebench/token_rounding.py:50-81 (SonicMoE Algorithm 4) from its behaviour:
plain top-k routing, then every expert's token count is moved to the nearest multiple of the tile (ties
down, never above the largest multiple that fits in T) by dropping its lowest-scoring picks or adding the
highest-scoring tokens that did not pick it; equal scores rank in token order; each token's weights are
its kept scores renormalised. Pinned against outputs of the reference itself (tests/golden/rounding.npz).
"""

from __future__ import annotations

import torch


def round_counts(counts: torch.Tensor, tile: int, max_count: int) -> torch.Tensor:
    """Nearest multiple of `tile`, ties down, at most max_count // tile * tile (reference: token_rounding.py:50-55)."""
    low = counts // tile * tile
    high = low + tile * (counts % tile > 0)
    nearest = torch.where(high - counts < counts - low, high, low)
    return nearest.clamp(max=max_count // tile * tile)


def token_rounding(scores: torch.Tensor, k: int, tile: int = 128):
    """scores [T, E] -> (token [N], expert [N], weight [N]) in token-major, expert-ascending order
    (reference: token_rounding.py:58-81, written out per expert instead of with a column sort)."""
    num_tokens, num_experts = scores.shape
    picks = scores.topk(k, dim=1).indices
    picked = torch.zeros(num_tokens, num_experts, dtype=torch.bool)
    picked[torch.arange(num_tokens)[:, None], picks] = True
    target = round_counts(picked.sum(dim=0), tile, num_tokens)
    keep = picked.clone()
    for e in range(num_experts):
        f, want = int(picked[:, e].sum()), int(target[e])
        if want == f:
            continue
        column = scores[:, e]
        if want < f:  # keep the `want` best picks
            candidates = torch.nonzero(picked[:, e]).flatten()
            order = torch.sort(column[candidates], descending=True, stable=True).indices
            keep[candidates[order[want:]], e] = False
        else:         # add the best tokens that did not pick e
            candidates = torch.nonzero(~picked[:, e]).flatten()
            order = torch.sort(column[candidates], descending=True, stable=True).indices
            keep[candidates[order[: want - f]], e] = True
    token, expert = keep.nonzero(as_tuple=True)
    raw = scores[token, expert]
    total = torch.zeros(num_tokens, dtype=raw.dtype).index_add_(0, token, raw)
    return token, expert, (raw / total[token]).float()
