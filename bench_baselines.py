"""Library-kernel pipelines for the same MoE layer, timed the same way, as context for the numbers.

These are NOT the product path and nothing in the package calls them: they answer "what does the
same layer cost on this GPU with stock PyTorch kernels". The reference compares itself with the same
kinds of pipelines (bench/bench_moe.py and sparsebench/baselines.py:255-290: per-expert loop, padded
bmm and torch._grouped_mm; its other competitors, stk / grouped_gemm / ScatterMoE, are third-party
packages that are not installed here).

  per_expert_loop   sort copies by expert, one cuBLAS matmul pair per expert (needs the per-expert
                    counts on the host: one sync per layer), gate-weighted sum
  padded_bmm        GShard / Switch style: every expert padded to the busiest one's row count, two
                    batched matmuls over [E, capacity, .] (needs that maximum on the host: one sync)
  grouped_mm        torch._grouped_mm for both matmuls (offsets stay on the device, no sync)

    python bench_baselines.py [workload ...]      # one JSON line per pipeline and workload
    python bench_baselines.py --reference-gpu [workload ...]
                                                  # the REFERENCE's own CUDA kernels on this GPU (below)

bench.py calls measure() for its `library_baselines` key and runs the --reference-gpu form as a child
process for its `reference_gpu_kernels` key.

--reference-gpu: the reference ships CUDA kernels for sm_80 / sm_90a only (mma.sync, cp.async, ldmatrix).
oracle/build_ref_ext.py compiles those sources, unmodified, for sm_100; here its four entry points are
chained exactly as the reference's moe_forward chains them (sparsebench/moe.py:44-55: routing, SDD+GELU,
DSD version 5, PyTorch gather + weighted sum) and timed like everything else. This is the reference's
GPU path on the same machine: a comparison row, in a process of its own, never part of the product path.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from sparsebench_b200.timing import l2_flush_buffer, time_ms  # noqa: E402
from sparsebench_b200.workloads import CONFIGS, make_layer  # noqa: E402


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


def padded_bmm(x, expert_idx, expert_weight, w1, w2) -> torch.Tensor:
    num_experts = w1.shape[0]
    xs, order, counts = _sorted_copies(x, expert_idx, num_experts)
    capacity = int(counts.max().item())  # host sync: the padded shape depends on the busiest expert
    starts = torch.cumsum(counts, 0) - counts
    expert_of_row = torch.repeat_interleave(torch.arange(num_experts, device=x.device), counts,
                                            output_size=xs.shape[0])
    slot = torch.arange(xs.shape[0], device=x.device) - starts[expert_of_row]
    padded = xs.new_zeros(num_experts, capacity, xs.shape[1])
    padded[expert_of_row, slot] = xs
    y = torch.bmm(F.gelu(torch.bmm(padded, w1)), w2)
    return _combine(y[expert_of_row, slot], order, expert_weight, x.shape[0])


def grouped_mm(x, expert_idx, expert_weight, w1, w2) -> torch.Tensor:
    xs, order, counts = _sorted_copies(x, expert_idx, w1.shape[0])
    offs = torch.cumsum(counts, 0).to(torch.int32)
    h = F.gelu(torch._grouped_mm(xs, w1, offs=offs))
    y = torch._grouped_mm(h, w2, offs=offs)
    return _combine(y, order, expert_weight, x.shape[0])


PIPELINES = {"per_expert_loop": per_expert_loop, "padded_bmm": padded_bmm, "grouped_mm": grouped_mm}


def measure(cfg, dev, flush: torch.Tensor, ours: torch.Tensor | None = None, iters: int = 20,
            pipelines: dict | None = None) -> dict:
    """{pipeline: {ms, useful_tflops, max_abs_diff_vs_ours} or {unavailable}} for one workload whose
    inputs `dev` are already on the GPU. Eager calls, CUDA events, L2 flushed before every call."""
    args = (dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    out: dict = {}
    for label, fn in (pipelines or PIPELINES).items():
        row: dict = {}
        try:
            result = fn(*args)
            if ours is not None:
                row["max_abs_diff_vs_ours"] = float((result.float() - ours.float()).abs().max())
            del result
            ms = time_ms(lambda: fn(*args), flush, warmup=3, iters=iters)
            row.update({"ms": ms, "useful_tflops": cfg.useful_flops / (ms * 1e-3) / 1e12})
        except Exception as exc:  # noqa: BLE001 - a baseline that cannot run says why
            row = {"unavailable": repr(exc)[:200]}
            torch.cuda.empty_cache()
        out[label] = row
    return out


def reference_gpu_forward(ext):
    """The reference's layer over its own extension module `ext` (same stage order and the same PyTorch
    combine as sparsebench/moe.py:44-55)."""
    def forward(x, expert_idx, expert_weight, w1, w2) -> torch.Tensor:
        num_experts, d_model, ffn_dim = w1.shape
        (_, _, row_token, copy_row, row_block_expert, row_offsets, col_indices, _) = ext.build_topology_cuda(
            expert_idx, num_experts, ffn_dim, 128)
        h = ext.sdd_cuda(x, w1, row_token, row_block_expert, row_offsets, col_indices.numel(), True)
        y = ext.dsd_cuda(h, w2.view(num_experts * ffn_dim, d_model), row_offsets, col_indices, 5)
        num_tokens, k = expert_idx.shape
        rows = y[copy_row.long()].view(num_tokens, k, d_model)
        return (rows.float() * expert_weight.float()[..., None]).sum(dim=1).to(x.dtype)

    return forward


def reference_gpu_main(names: list[str]) -> None:
    """One JSON line per workload: the reference's own kernels (built for sm_100) on this GPU, eagerly
    and as one CUDA-graph replay per step, plus the largest difference from this library's output."""
    from oracle.build_ref_ext import load_ref_ext
    from sparsebench_b200 import moe_forward

    ext, why = load_ref_ext()
    flush = l2_flush_buffer() if ext is not None else None
    for name in names or ["fine_grained"]:
        line: dict = {"workload": name, "pipeline": "reference CUDA kernels built for sm_100"}
        if ext is None:
            line["unavailable"] = why
            print(json.dumps(line), flush=True)
            continue
        try:
            cfg = CONFIGS[name]
            dev = make_layer(cfg).to("cuda")
            args = (dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
            forward = reference_gpu_forward(ext)
            out = forward(*args)
            line["arch_probe"] = int(ext.arch_probe(1)[0].item())
            line["max_abs_diff_vs_this_library"] = float((out.float() - moe_forward(*args).float()).abs().max())
            line["eager_ms"] = time_ms(lambda: forward(*args), flush, warmup=3, iters=20)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                forward(*args)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                forward(*args)
            ms = time_ms(graph.replay, flush, warmup=3, iters=20)
            line.update({"graph_ms": ms, "useful_tflops": cfg.useful_flops / (ms * 1e-3) / 1e12})
            del graph, dev, args, out
            torch.cuda.empty_cache()
        except Exception as exc:  # noqa: BLE001 - a comparison row that cannot run says why
            line["unavailable"] = repr(exc)[:300]
        print(json.dumps(line), flush=True)


def main(argv: list[str]) -> None:
    if argv and argv[0] == "--reference-gpu":
        reference_gpu_main(argv[1:])
        return
    from sparsebench_b200 import moe_forward

    names = argv or ["fine_grained", "mixtral_like"]
    flush = l2_flush_buffer()
    for name in names:
        cfg = CONFIGS[name]
        dev = make_layer(cfg).to("cuda")
        ours = moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
        rows = measure(cfg, dev, flush, ours, pipelines={"sparsebench_b200.moe_forward": moe_forward, **PIPELINES})
        for label, row in rows.items():
            print(json.dumps({"workload": name, "pipeline": label, **row}), flush=True)
        del dev, ours
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main(sys.argv[1:])
