"""Token rounding without a host sync: the reference's sparsebench/token_rounding.py surface on the device.

The reference builds the rounded routing with PyTorch ops and one host sync (nonzero) and hands the flat
list to moe_forward_assigned. Here three small kernels build the same list at its worst-case length, with
unused entries marked by expert -1, so that router scores -> rounded routing -> layer runs with no host
sync at all and can be captured in a CUDA graph.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from sparsebench_b200 import _C
from sparsebench_b200.moe import moe_forward_assigned


@dataclass(frozen=True)
class DeviceAssignments:
    """A routing as a flat, worst-case sized list on the device: copy c sends token[c] to expert[c] with
    weight[c]; entries at and past count[0] have expert -1 (reference: token_rounding.py:30-36)."""

    token: torch.Tensor  # [cap] int32
    expert: torch.Tensor  # [cap] int32, -1 = unused entry
    weight: torch.Tensor  # [cap] float32
    count: torch.Tensor  # [1] int32, entries in use

    def trimmed(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Syncs. (token, expert, weight) cut to the entries in use, as int64 / int64 / float32."""
        n = int(self.count.item())
        return self.token[:n].long(), self.expert[:n].long(), self.weight[:n]


def token_rounding(scores: torch.Tensor, k: int, tile: int = 128) -> DeviceAssignments:
    """scores [T, E] fp32 router probabilities (CUDA) -> routing in which every expert's token count is a
    multiple of `tile`. No host sync."""
    if scores.dim() != 2 or not 0 < k <= scores.shape[1]:
        raise ValueError(f"need [T, E] scores with 0 < k <= E, got {tuple(scores.shape)} and k={k}")
    return DeviceAssignments(*_C.token_rounding_cuda(scores.float().contiguous(), k, tile))


def moe_forward_rounded(x: torch.Tensor, scores: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, k: int = 2,
                        tile: int = 128) -> torch.Tensor:
    """The layer on a token-rounded routing of `scores` [T, E]: rounding, routing, SDD, DSD and the combine,
    all enqueued without the host ever learning how many assignments survived."""
    routed = token_rounding(scores, k, tile)
    return moe_forward_assigned(x, routed.token, routed.expert, routed.weight, w1, w2)
