"""The expert-parallel arm of bench.py: one rank per GPU under torchrun (or a single process for
world size 1). Weak scaling: every rank brings T tokens, the E experts are split over the ranks.

Timing: CUDA events around every step on the launching stream, 256 MiB written and read back before
every step to flush L2, a barrier and a device synchronise on both sides of the timed region, per-rank sums
reduced with MAX. The step is one CUDA-graph replay when the collectives can be captured, else
eager launches (config.launch says which).
"""

from __future__ import annotations

import json
import math
import os
import sys

import torch
import torch.distributed as dist

from sparsebench_b200.ep import ExpertParallelMoE
from sparsebench_b200.timing import flush_l2, l2_flush_buffer
from sparsebench_b200.workloads import CONFIGS, make_layer

NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy on this pool; 900 nominal

# Micro-batches per step by rank count, where measured to pay (the owner's matmuls tensor-bound and the
# exchange a large share of the step); elsewhere the step runs whole.
# 8 ranks (16 experts each, the busiest rank tensor-bound): 0.469 ms whole, 0.427 ms in two parts; 2 ranks (64
# experts each, HBM-bound): 0.335 ms whole, 0.465 ms in two parts.
DEFAULT_MICRO_BATCHES: dict[int, int] = {8: 2}



def _timed_steps(step, flush: torch.Tensor, warmup: int, steps: int, world: int) -> float:
    """Mean ms per step, max over ranks."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    pairs = []
    aligned = torch.zeros(1, device=flush.device)
    for _ in range(steps):
        flush_l2(flush)
        if world > 1:
            # The ranks' flushes do not take exactly the same time; without this the rank that finishes
            # first would spend the difference waiting inside its timed step, at the first exchange.
            dist.all_reduce(aligned)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        step()
        end.record()
        pairs.append((start, end))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    total = torch.tensor([sum(s.elapsed_time(e) for s, e in pairs)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    return float(total.item()) / steps


def _pipelined_e2e_ms(step, result_of, dev_inputs, host_inputs, warmup: int, steps: int, world: int) -> float:
    """Mean ms per step, max over ranks, of the step fed from pinned HOST buffers when consecutive steps
    overlap the way a serving loop runs them: three streams (copy in, step, copy out) and two sets of
    staging buffers. `step` reads fixed device tensors (a captured graph does), so the compute stream
    first copies the staged inputs into them (device to device, a few us) and the result out into the
    set's staging tensor. Every step's host->device and device->host copies are inside the timed region."""
    device = dev_inputs[0].device
    copy_in, compute, copy_out = (torch.cuda.Stream(device) for _ in range(3))
    sets = []
    for _ in range(2):
        sets.append({
            "in": [torch.empty_like(t) for t in dev_inputs],
            "out": torch.empty_like(dev_inputs[0]),
            "host_out": torch.empty(dev_inputs[0].shape, dtype=dev_inputs[0].dtype).pin_memory(),
            "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "copied": torch.cuda.Event(),
        })

    def run(n: int) -> None:
        for i in range(n):
            b = sets[i % 2]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(b["computed"])  # the step that last read this set's inputs is done
                for staged, host in zip(b["in"], host_inputs):
                    staged.copy_(host, non_blocking=True)
                b["loaded"].record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(b["loaded"])
                compute.wait_event(b["copied"])  # this set's result tensor has been read out
                for fixed, staged in zip(dev_inputs, b["in"]):
                    fixed.copy_(staged, non_blocking=True)
                b["out"].copy_(result_of(step()), non_blocking=True)
                b["computed"].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(b["computed"])
                b["host_out"].copy_(b["out"], non_blocking=True)
                b["copied"].record(copy_out)

    torch.cuda.synchronize(device)
    run(max(warmup, 4))
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(copy_in)
    run(steps)
    for stream in (copy_in, compute):
        copy_out.wait_stream(stream)
    end.record(copy_out)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    total = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    return float(total.item()) / steps


def run(args, metric: str, peaks: tuple[float, float, str], clock_sampler_cls) -> None:
    """Measures the expert-parallel step on every rank; rank 0 prints the JSON line."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    line = measure(args, metric, peaks, clock_sampler_cls, world, rank, local)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        # Leave without tearing the communicator down: destroying it while a captured graph still
        # holds its collectives has been seen to block forever. Every rank has printed and
        # synchronised by now, so a hard exit loses nothing.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def measure(args, metric: str, peaks: tuple[float, float, str], clock_sampler_cls, world: int, rank: int,
            local: int) -> dict:
    """One full measurement of the expert-parallel step; returns the JSON line (meaningful on rank 0)."""
    device = torch.device("cuda", local)
    cfg = CONFIGS[args.workload or "expert_parallel"]
    if cfg.num_experts % world != 0:
        raise SystemExit(f"{cfg.num_experts} experts do not split over {world} ranks")
    per_rank = cfg.num_experts // world
    mine = range(rank * per_rank, (rank + 1) * per_rank)
    layer_in = make_layer(cfg, seed=0, token_seed=rank, experts=mine)
    dev = layer_in.to(device)
    # Rows per (source, destination) pair. T*k can never overflow but sends N times the payload; a
    # factor over the even share T*k/N covers skewed routing (the busiest of 8 ranks draws about 2.3x
    # its share under Zipf(1.2)). An overflow is detected on the device and fails the run below.
    n_copies = cfg.num_tokens * cfg.k
    factor = getattr(args, "ep_capacity_factor", 3.0)
    capacity = min(n_copies, int(math.ceil(factor * n_copies / world / 128.0)) * 128)
    exchange = getattr(args, "ep_exchange", "peer") if world > 1 else "nccl"
    # Micro-batches pipelined over streams (peer exchange): 0 = this build's default for the rank count.
    micro_batches = getattr(args, "ep_micro_batches", 0) or DEFAULT_MICRO_BATCHES.get(world, 1)
    moe = None
    if exchange == "peer":
        # Rows stored straight into the owner's memory: only real rows travel, so the capacity can be
        # the exact worst case. If the buffers cannot be mapped on this machine every rank falls back.
        try:
            moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=n_copies, exchange="peer",
                                    fuse_return=not getattr(args, "ep_unfused_return", False),
                                    micro_batches=micro_batches)
            mapped = torch.ones(1, device=device)
        except Exception as exc:  # noqa: BLE001 - reported in the JSON line
            mapped = torch.zeros(1, device=device)
            peer_error = repr(exc)
        dist.all_reduce(mapped, op=dist.ReduceOp.MIN)
        if mapped.item() == 0:
            moe, exchange = None, "nccl (peer mapping failed: %s)" % locals().get("peer_error", "on another rank")
        else:
            capacity = n_copies
    if moe is None:
        moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=capacity)
    flush = l2_flush_buffer(device)
    hbm_gbs, bf16_tflops, peak_kind = peaks

    out = moe(dev.x, dev.expert_idx, dev.expert_weight)
    torch.cuda.synchronize()
    overflow = moe.status.clone()
    if world > 1:
        dist.all_reduce(overflow, op=dist.ReduceOp.MAX)
    if int(overflow.item()) != 0:
        raise SystemExit(f"expert-parallel exchange overflowed {capacity} rows per pair: raise --ep-capacity-factor")

    # ---- value: graph replay if the collectives capture, else eager --------------------------------
    launch = "eager launches (graph capture of the collectives was refused)"
    graph_out = None
    step = lambda: moe(dev.x, dev.expert_idx, dev.expert_weight)  # noqa: E731
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            moe(dev.x, dev.expert_idx, dev.expert_weight)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = moe(dev.x, dev.expert_idx, dev.expert_weight)
        graph.replay()
        torch.cuda.synchronize()
        if not torch.equal(graph_out, out):
            raise RuntimeError("graph replay and eager launch disagree")
        step, launch = graph.replay, "one CUDA-graph replay per step"
    except RuntimeError as exc:
        if "disagree" in str(exc):
            raise
        torch.cuda.synchronize()

    # Kernels of this library per step: sort, plan, (pack | push counts + push rows + barrier),
    # slot experts, routing (1 launch, 3 beyond 262144 slots), SDD, DSD, (pack | [push rows +] barrier), combine.
    route_launches = 1 if world * moe.capacity <= 262144 else 3
    fused_return = moe.peer is not None and moe.fuse_return
    launches_per_step = (12 if moe.peer is not None else 8) + route_launches - (1 if fused_return else 0)
    if moe.micro_batches > 1:
        launches_per_step = launches_per_step * moe.micro_batches + 1  # every part is a whole step, plus the concatenation
    with clock_sampler_cls(local) as clocks:
        ms_per_step = _timed_steps(step, flush, args.warmup, args.steps, world)
    value = world * cfg.useful_flops / (ms_per_step * 1e-3) / 1e12

    # ---- e2e: public API with host buffers -----------------------------------------------------------
    host_x, host_idx, host_w = (t.pin_memory() for t in (layer_in.x, layer_in.expert_idx, layer_in.expert_weight))
    host_out = torch.empty_like(layer_in.x).pin_memory()
    def e2e_step() -> None:
        # `step` is the captured graph (or the eager call) over dev.x / dev.expert_idx / dev.expert_weight.
        dev.x.copy_(host_x, non_blocking=True)
        dev.expert_idx.copy_(host_idx, non_blocking=True)
        dev.expert_weight.copy_(host_w, non_blocking=True)
        result = step()
        host_out.copy_(graph_out if result is None else result, non_blocking=True)

    e2e_latency_ms = _timed_steps(e2e_step, flush, args.warmup, args.steps, world)  # one step alone, nothing overlapped
    e2e_ms = _pipelined_e2e_ms(step, lambda result: graph_out if result is None else result,
                               (dev.x, dev.expert_idx, dev.expert_weight), (host_x, host_idx, host_w), args.warmup,
                               args.steps, world)
    h2d = sum(t.numel() * t.element_size() for t in (host_x, host_idx, host_w))
    d2h = host_out.numel() * host_out.element_size()

    # ---- per-stage times on this rank (eager, an event at every stage mark) ---------------------------
    # With micro-batches the stages of the parts interleave; the breakdown (and the roofline of the
    # dominant matmul) is then taken on the same step run whole.
    timed_moe = moe
    if moe.micro_batches > 1:
        moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=n_copies, exchange="peer",
                                fuse_return=timed_moe.fuse_return)
    names: list[str] = []
    sums: dict[str, float] = {}
    iters = max(5, min(args.steps, 30))
    for it in range(iters + 2):
        flush_l2(flush)
        events = [torch.cuda.Event(enable_timing=True)]
        events[0].record()
        seen: list[str] = []

        def mark(stage: str) -> None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            events.append(ev)
            seen.append(stage)

        moe(dev.x, dev.expert_idx, dev.expert_weight, mark=mark)
        torch.cuda.synchronize()
        if it >= 2:
            names = seen
            for i, stage in enumerate(seen):
                sums[stage] = sums.get(stage, 0.0) + events[i].elapsed_time(events[i + 1])
    stage_ms = {s: sums[s] / iters for s in names}

    rows = int(moe.last.owner_layout.padded_offsets[-1].item())  # live padded rows on this rank
    received = int(moe.last.recv_counts.sum().item())
    # SDD stores, and DSD loads and stores, whole groups of 32 rows only where one holds a real row.
    per_expert = moe.last.recv_counts.sum(dim=0)
    rows_moved = int(((per_expert + 31) // 32 * 32).sum().item())
    weight_bytes = per_rank * cfg.d_model * cfg.ffn_dim * 2
    sdd_bytes = received * cfg.d_model * 2 + weight_bytes + rows_moved * cfg.ffn_dim * 2
    dsd_bytes = rows_moved * cfg.ffn_dim * 2 + weight_bytes + rows_moved * cfg.d_model * 2
    gemm_ms = {"sdd": stage_ms["SDD + GELU (fused)"], "dsd": stage_ms["DSD"]}
    gemm_bytes = {"sdd": sdd_bytes, "dsd": dsd_bytes}
    dominant = max(gemm_ms, key=gemm_ms.get)
    t_dom = gemm_ms[dominant] * 1e-3
    exec_flops = 2 * rows * cfg.d_model * cfg.ffn_dim
    if gemm_bytes[dominant] / (hbm_gbs * 1e9) >= exec_flops / (bf16_tflops * 1e12):
        achieved = gemm_bytes[dominant] / t_dom / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs}
    else:
        achieved = exec_flops / t_dom / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": bf16_tflops, "unit": "TFLOP/s",
                    "frac": achieved / bf16_tflops}
    payload = (world - 1) / world * cfg.num_tokens * cfg.k * cfg.d_model * 2  # useful bytes per direction
    roofline.update({
        "kernel": f"bsr_gemm_kernel<{dominant}> on rank 0", "peak_source": peak_kind, "launch_ms": gemm_ms[dominant],
        "algorithmic_bytes": gemm_bytes[dominant], "live_rows": rows, "rows_moved": rows_moved, "traffic": None, "stages_ms": stage_ms,
        "all_to_all": {"useful_bytes_per_direction": payload,
                       "sent_bytes_per_direction": payload if moe.peer is not None else world * moe.capacity * cfg.d_model * 2,
                       "time_at_measured_nvlink_ms": payload / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3},
    })

    line = {
        "metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name, "tokens_per_gpu": cfg.num_tokens, "d_model": cfg.d_model,
                   "ffn_dim": cfg.ffn_dim, "experts": cfg.num_experts, "experts_per_gpu": per_rank, "top_k": cfg.k,
                   "routing": cfg.routing, "parallelism": f"ep{world}", "capacity_rows_per_pair": moe.capacity,
                   "exchange": exchange, "return_leg": "stored by the DSD epilogue" if fused_return else "separate kernel",
                   "micro_batches": timed_moe.micro_batches,
                   "launch": launch, "l2": "256 MiB written and read back before every step (L2 cold and clean)",
                   "frac_of_bf16_peak": value / world / bf16_tflops},
        "clocks": clocks.summary(),
        "e2e": {"value": world * cfg.useful_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "steps pipelined over three streams (copy in, step, copy out), two sets of staging buffers; "
                       "every step's H2D and D2H copies are inside the timed region",
                "single_step_latency_ms": e2e_latency_ms},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": roofline,
    }
    return line
