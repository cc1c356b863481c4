"""Library-kernel pipelines for the same MoE layer, timed the same way, as context for the numbers.

These are NOT the product path and nothing in the package calls them: they answer "what does the
same layer cost on this GPU with stock PyTorch kernels". The reference compares itself with the same
kinds of pipelines (bench/bench_moe.py: per-expert loop and torch._grouped_mm; its other competitors,
stk / grouped_gemm / ScatterMoE, are third-party packages that are not installed here).

  per_expert_loop   sort copies by expert, one cuBLAS matmul pair per expert (needs the per-expert
                    counts on the host: one sync per layer), gate-weighted scatter-add
  grouped_mm        the same with torch._grouped_mm for both matmuls (offsets stay on the device)

    python -m sparsebench_b200.baselines [workload ...]      # one JSON line per pipeline and workload
"""

from __future__ import annotations

import json
import sys

import torch
import torch.nn.functional as F

from sparsebench_b200.timing import l2_flush_buffer, time_ms
from sparsebench_b200.workloads import CONFIGS, make_layer


def _sorted_copies(x: torch.Tensor, expert_idx: torch.Tensor, num_experts: int):
    flat = expert_idx.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    token = order // expert_idx.shape[1]
    return x[token], order, counts


def _combine(y_sorted: torch.Tensor, order: torch.Tensor, expert_weight: torch.Tensor, num_tokens: int) -> torch.Tensor:
    k = expert_weight.shape[1]
    rows = torch.empty_like(y_sorted)
    rows[order] = y_sorted  # back to copy order
    return (rows.view(num_tokens, k, -1).float() * expert_weight.float()[..., None]).sum(dim=1).to(y_sorted.dtype)


def per_expert_loop(x, expert_idx, expert_weight, w1, w2) -> torch.Tensor:
    xs, order, counts = _sorted_copies(x, expert_idx, w1.shape[0])
    y = torch.empty_like(xs)
    start = 0
    for e, n in enumerate(counts.tolist()):  # host sync: the loop needs the counts
        if n:
            y[start : start + n] = F.gelu(xs[start : start + n] @ w1[e]) @ w2[e]
            start += n
    return _combine(y, order, expert_weight, x.shape[0])


def grouped_mm(x, expert_idx, expert_weight, w1, w2) -> torch.Tensor:
    xs, order, counts = _sorted_copies(x, expert_idx, w1.shape[0])
    offs = torch.cumsum(counts, 0).to(torch.int32)
    h = F.gelu(torch._grouped_mm(xs, w1, offs=offs))
    y = torch._grouped_mm(h, w2, offs=offs)
    return _combine(y, order, expert_weight, x.shape[0])


PIPELINES = {"per_expert_loop": per_expert_loop, "grouped_mm": grouped_mm}


def main(argv: list[str]) -> None:
    from sparsebench_b200 import moe_forward

    names = argv or ["fine_grained", "mixtral_like"]
    flush = l2_flush_buffer()
    for name in names:
        cfg = CONFIGS[name]
        dev = make_layer(cfg).to("cuda")
        args = (dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
        ours = moe_forward(*args)
        rows = [("sparsebench_b200.moe_forward", moe_forward)] + list(PIPELINES.items())
        for label, fn in rows:
            line = {"workload": name, "pipeline": label}
            try:
                out = fn(*args)
                line["max_abs_diff_vs_ours"] = float((out.float() - ours.float()).abs().max())
                ms = time_ms(lambda: fn(*args), flush, warmup=3, iters=20)
                line.update({"ms": ms, "useful_tflops": cfg.useful_flops / (ms * 1e-3) / 1e12})
            except Exception as exc:  # noqa: BLE001 - a baseline that cannot run says why
                line["unavailable"] = repr(exc)[:200]
            print(json.dumps(line), flush=True)
        del dev, args, ours
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main(sys.argv[1:])
