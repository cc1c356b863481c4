"""Benchmark of the sync-free MoE forward layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one forward pass of the layer (routing -> SDD+GELU -> DSD -> combine) over one batch
of synthetic tokens. Metric: useful TFLOP/s = 4*T*k*D*F / time (padding rows are waste, not work),
with ms per step next to it.

  N = 1   workload "fine_grained": T=4096, D=1024, F=4096, E=64, top-2, uniform routing, bf16.
  N > 1   workload "expert_parallel": E=128 experts sharded over the N GPUs, T=4096 tokens per GPU,
          D=2048, F=2048, top-2, permuted-Zipf routing; token dispatch/return by all-to-all (NCCL).
          Launched by torchrun, one rank per GPU. Weak scaling: per-GPU tokens are fixed.

Prints ONE JSON line (rank 0):
  value      whole-job TFLOP/s with inputs resident in HBM, one CUDA-graph replay per step, CUDA
             events around every step, L2 flushed before every step, max over ranks
  e2e        the same metric through the public API (moe_forward) with HOST buffers: every step
             copies its tokens, routing and gates from pinned host memory and reads the output
             back, all inside the timed region; consecutive steps overlap on three streams the way
             a serving loop runs them (the unoverlapped single-step latency is reported beside it)
  roofline   the dominant kernel's algorithmic bytes / its measured duration against the measured
             HBM copy bandwidth of this pool (MEASURED_PEAKS.json, else the stated fallback)
  cpu_baseline  the fp32 CPU oracle of the same layer timed on this machine's host cores

--impl reference times only that CPU implementation and prints its own line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from sparsebench_b200.workloads import CONFIGS, LayerConfig, make_layer  # noqa: E402

METRIC = "moe_fwd_useful_tflops"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
# profiles/bsr_gemm_kernel_fine_grained.md (same workload, same kernels).
NCU_TRAFFIC_BYTES = {("fine_grained", "sdd"): 576.8e6, ("fine_grained", "dsd"): 619.1e6}
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks() -> tuple[float, float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.005) -> None:
        self.period_s = period_s
        self.samples: list[int] = []
        self.reasons = 0
        self.max_mhz = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[device_index]) if visible and visible.replace(",", "").isdigit() else device_index
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # NVML missing: report empty clocks rather than fail the benchmark
            self._nvml = None

    def _run(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                self.reasons |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                pass
            time.sleep(self.period_s)

    def __enter__(self) -> "ClockSampler":
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        names = []
        if self._nvml is not None:
            nv = self._nvml
            table = {
                "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
                "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
            }
            names = [k for k, bit in table.items() if self.reasons & bit]
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz or None,
            "reasons": names,
            "samples": len(self.samples),
        }


def pipelined_e2e_ms(forward, host_inputs, weights, warmup: int, steps: int) -> float:
    """ms per step of `forward` fed from pinned HOST buffers when consecutive steps overlap the way a
    serving loop runs them: step i+1's inputs are copied in while step i computes and step i-1's
    result is copied out (three streams, two sets of device buffers, the layer of each set captured
    once as a CUDA graph and replayed, so that the host only enqueues copies and one graph launch per
    step). Every step's host->device and device->host copies are inside the timed region; the
    weights (1 GB, far larger than L2) are re-streamed from HBM by every step."""
    host_x, host_idx, host_w = host_inputs
    device = weights[0].device
    copy_in, compute, copy_out = (torch.cuda.Stream(device) for _ in range(3))
    sets = []
    for _ in range(2):
        b = {
            "x": torch.empty(host_x.shape, dtype=host_x.dtype, device=device),
            "idx": torch.empty(host_idx.shape, dtype=host_idx.dtype, device=device),
            "w": torch.empty(host_w.shape, dtype=host_w.dtype, device=device),
            "out": torch.empty(host_x.shape, dtype=host_x.dtype).pin_memory(),
            "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "copied": torch.cuda.Event(),
        }
        b["x"].copy_(host_x)
        b["idx"].copy_(host_idx)
        b["w"].copy_(host_w)
        torch.cuda.synchronize(device)
        with torch.cuda.stream(compute):
            forward(b["x"], b["idx"], b["w"], *weights)  # one-time set-up outside the capture
        torch.cuda.synchronize(device)
        b["graph"] = torch.cuda.CUDAGraph()
        with torch.cuda.graph(b["graph"], stream=compute):
            b["result"] = forward(b["x"], b["idx"], b["w"], *weights)
        sets.append(b)

    def run(n: int) -> None:
        for i in range(n):
            b = sets[i % 2]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(b["computed"])  # the layer that last read this buffer set is done
                b["x"].copy_(host_x, non_blocking=True)
                b["idx"].copy_(host_idx, non_blocking=True)
                b["w"].copy_(host_w, non_blocking=True)
                b["loaded"].record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(b["loaded"])
                compute.wait_event(b["copied"])  # the graph's output buffer has been read out
                b["graph"].replay()
                b["computed"].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(b["computed"])
                b["out"].copy_(b["result"], non_blocking=True)
                b["copied"].record(copy_out)

    torch.cuda.synchronize(device)
    run(max(warmup, 4))
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(copy_in)
    run(steps)
    for stream in (copy_in, compute):
        copy_out.wait_stream(stream)
    end.record(copy_out)
    torch.cuda.synchronize(device)
    return start.elapsed_time(end) / steps


def live_rows(expert_idx: torch.Tensor, num_experts: int, granule: int = 128) -> int:
    """Rows of the layout after rounding every expert's copies up to `granule`: 128 is what the tensor
    cores execute (whole row blocks), 32 what SDD stores and DSD loads and stores in the layer (groups
    of 32 rows that are all padding are skipped)."""
    counts = torch.bincount(expert_idx.reshape(-1), minlength=num_experts)
    return int(((counts + granule - 1) // granule * granule).sum())


def cpu_baseline(cfg: LayerConfig, layer, budget_s: float = 20.0) -> dict:
    """The fp32 CPU oracle (a port of the reference's moe_reference) on this machine's host cores."""
    from oracle import moe as oracle_moe

    x, w = layer.x.float(), layer.expert_weight.float()
    w1, w2 = layer.w1.float(), layer.w2.float()
    times = []
    started = time.perf_counter()
    for i in range(7):
        t0 = time.perf_counter()
        oracle_moe.moe_reference(x, layer.expert_idx, w, w1, w2)
        dt = time.perf_counter() - t0
        if i >= 2:
            times.append(dt)
        if time.perf_counter() - started > budget_s and len(times) >= 1:
            break
    med = statistics.median(times)
    return {
        "value": cfg.useful_flops / med / 1e12,
        "unit": "TFLOP/s",
        "ms_per_step": med * 1e3,
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": "port",
        "sample": f"whole {cfg.name} layer in fp32, median of {len(times)} runs after 2 warm-up runs",
    }


def run_reference_arm(args: argparse.Namespace) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = CONFIGS[args.workload or ("fine_grained" if args.gpus == 1 else "expert_parallel")]
    if args.gpus > 1:  # the CPU arm computes the global batch of all ranks' tokens
        cfg = LayerConfig(cfg.name, cfg.num_tokens * args.gpus, cfg.d_model, cfg.ffn_dim, cfg.num_experts, cfg.routing)
    from oracle import moe as oracle_moe

    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm is alone on the host, so it takes
    # every core the process may run on.
    torch.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    layer = make_layer(cfg, seed=0)
    x, w = layer.x.float(), layer.expert_weight.float()
    w1, w2 = layer.w1.float(), layer.w2.float()
    # A step here is a bounded sample: the first `sample_tokens` tokens of the batch through the
    # whole layer, so that steps + warmup stay within a few minutes on the host cores.
    sample_tokens = min(cfg.num_tokens, 4096)
    xs, idx, ws = x[:sample_tokens], layer.expert_idx[:sample_tokens], w[:sample_tokens]
    steps, warmup = min(args.steps, 10), min(args.warmup, 2)
    for _ in range(warmup):
        oracle_moe.moe_reference(xs, idx, ws, w1, w2)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        oracle_moe.moe_reference(xs, idx, ws, w1, w2)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    flops = 4 * sample_tokens * cfg.k * cfg.d_model * cfg.ffn_dim
    value = flops / sec / 1e12
    sample = f"{sample_tokens} of {cfg.num_tokens} tokens through the whole fp32 layer per step, {steps} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name, "tokens": cfg.num_tokens, "d_model": cfg.d_model, "ffn_dim": cfg.ffn_dim,
                   "experts": cfg.num_experts, "top_k": cfg.k, "routing": cfg.routing},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_single_gpu(args: argparse.Namespace) -> None:
    from sparsebench_b200 import _C, moe_forward, route_device
    from sparsebench_b200.spmm import combine, dsd, sdd
    from sparsebench_b200.timing import l2_flush_buffer, marginal_stage_times_ms, time_each_ms

    cfg = CONFIGS[args.workload or "fine_grained"]
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    layer = make_layer(cfg, seed=0)
    dev = layer.to(device)
    flush = l2_flush_buffer(device)
    hbm_gbs, bf16_tflops, peak_kind = measured_peaks()

    # ---- correctness gate on a subset of rows before timing anything -------------------------------
    out = moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    torch.cuda.synchronize()
    if int(_C.device_status(device).item()) != 0:
        raise RuntimeError("device status is non-zero: a bounded device-side wait expired")

    # ---- value: graph replay, inputs resident in HBM ------------------------------------------------
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_out = moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    torch.cuda.synchronize()

    with ClockSampler(0) as clocks:
        torch.cuda.synchronize()
        step_ms = time_each_ms(graph.replay, flush, warmup=args.warmup, iters=args.steps)
        torch.cuda.synchronize()
    ms_per_step = sum(step_ms) / len(step_ms)
    value = cfg.useful_flops / (ms_per_step * 1e-3) / 1e12
    # The same with the flush buffer only written (the reference's flush): every step then starts with
    # 126 MB of dirty lines in L2 whose write-back the first matmul pays for. Reported beside the value.
    dirty_ms = time_each_ms(graph.replay, flush, warmup=3, iters=min(args.steps, 50), leave_l2_dirty=True)
    ms_per_step_dirty_l2 = sum(dirty_ms) / len(dirty_ms)
    if not torch.equal(graph_out, out):
        raise RuntimeError("graph replay and eager launch disagree")

    # ---- e2e: public API, host buffers, copies inside the timed region -------------------------------
    host_x, host_idx, host_w = (t.pin_memory() for t in (layer.x, layer.expert_idx, layer.expert_weight))
    host_out = torch.empty_like(layer.x).pin_memory()
    def e2e_step() -> None:
        # The layer is the graph captured above; its inputs live in dev.x / dev.expert_idx / dev.expert_weight.
        dev.x.copy_(host_x, non_blocking=True)
        dev.expert_idx.copy_(host_idx, non_blocking=True)
        dev.expert_weight.copy_(host_w, non_blocking=True)
        graph.replay()
        host_out.copy_(graph_out, non_blocking=True)

    e2e_ms = time_each_ms(e2e_step, flush, warmup=args.warmup, iters=args.steps)
    e2e_latency_ms = sum(e2e_ms) / len(e2e_ms)  # one step alone: copy in, layer, copy out, nothing overlapped
    e2e_ms_per_step = pipelined_e2e_ms(moe_forward, (host_x, host_idx, host_w), (dev.w1, dev.w2), args.warmup, args.steps)
    h2d = host_x.numel() * host_x.element_size() + host_idx.numel() * host_idx.element_size() + \
        host_w.numel() * host_w.element_size()
    d2h = host_out.numel() * host_out.element_size()

    # ---- per-kernel durations, each launch timed alone with events on the launching stream -----------
    topo = route_device(dev.expert_idx, cfg.num_experts, cfg.ffn_dim, 128)
    # As the layer runs them: padding-only groups of 32 rows neither stored nor loaded.
    h = sdd(dev.x, dev.w1, topo, skip_padding_rows=True)
    w2_cat = dev.w2.view(cfg.num_experts * cfg.ffn_dim, cfg.d_model)
    y = dsd(h, w2_cat, topo, version=5, skip_padding_rows=True)
    iters = max(5, min(args.steps, 50))
    # Each kernel's time in its place in the layer: differences between the graphs of the first j stages
    # (see marginal_stage_times_ms).
    def stage_route(state: dict) -> None:
        state["topo"] = route_device(dev.expert_idx, cfg.num_experts, cfg.ffn_dim, 128)

    def stage_sdd(state: dict) -> None:
        state["h"] = sdd(dev.x, dev.w1, state["topo"], skip_padding_rows=True)

    def stage_dsd(state: dict) -> None:
        state["y"] = dsd(state["h"], w2_cat, state["topo"], version=5, skip_padding_rows=True)

    def stage_combine(state: dict) -> None:
        state["out"] = combine(state["y"], dev.expert_weight, state["topo"])

    stage_ms = marginal_stage_times_ms([("routing", stage_route), ("sdd", stage_sdd), ("dsd", stage_dsd),
                                        ("combine", stage_combine)], flush, 3, iters)
    stage_timing = ("each kernel in its place in the layer: CUDA-graph replays of the first j stages (each closed by the "
                    "same one-element kernel), CUDA events around every replay, L2 flushed before it, stage j = "
                    "prefix j - prefix j-1")
    rows = live_rows(layer.expert_idx, cfg.num_experts)            # executed by the tensor cores
    rows_moved = live_rows(layer.expert_idx, cfg.num_experts, 32)  # stored / loaded
    n_copies = cfg.num_tokens * cfg.k
    weight_bytes = cfg.num_experts * cfg.d_model * cfg.ffn_dim * 2
    stage_bytes = {
        "sdd": cfg.num_tokens * cfg.d_model * 2 + weight_bytes + rows_moved * cfg.ffn_dim * 2,
        "dsd": rows_moved * cfg.ffn_dim * 2 + weight_bytes + rows_moved * cfg.d_model * 2,
        "combine": n_copies * cfg.d_model * 2 + n_copies * 6 + cfg.num_tokens * cfg.d_model * 2,
    }
    stage_flops = {"sdd": 2 * n_copies * cfg.d_model * cfg.ffn_dim, "dsd": 2 * n_copies * cfg.d_model * cfg.ffn_dim}
    dominant = max(("sdd", "dsd"), key=lambda s: stage_ms[s])
    t_dom = stage_ms[dominant] * 1e-3
    hbm_time = stage_bytes[dominant] / (hbm_gbs * 1e9)
    tensor_time = 4 * rows * cfg.d_model * cfg.ffn_dim / 2 / (bf16_tflops * 1e12)  # executed flops, padding included
    if hbm_time >= tensor_time:
        achieved = stage_bytes[dominant] / t_dom / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs}
    else:
        achieved = 2 * rows * cfg.d_model * cfg.ffn_dim / t_dom / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": bf16_tflops, "unit": "TFLOP/s",
                    "frac": achieved / bf16_tflops}
    roofline.update({
        "kernel": f"bsr_gemm_kernel<{dominant}>", "peak_source": f"{peak_kind} (MEASURED_PEAKS.json)" if peak_kind == "measured" else "fallback",
        "launch_ms": stage_ms[dominant], "algorithmic_bytes": stage_bytes[dominant], "live_rows": rows,
        "rows_moved": rows_moved, "traffic": NCU_TRAFFIC_BYTES.get((cfg.name, dominant)),
        "stages_ms": stage_ms, "stages_timing": stage_timing,
        "stages_frac_of_hbm_peak": {s: stage_bytes[s] / (stage_ms[s] * 1e-3) / 1e9 / hbm_gbs for s in stage_bytes},
        "stages_useful_tflops": {s: stage_flops[s] / (stage_ms[s] * 1e-3) / 1e12 for s in stage_flops},
    })

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": cfg.name, "tokens": cfg.num_tokens, "d_model": cfg.d_model, "ffn_dim": cfg.ffn_dim,
                   "experts": cfg.num_experts, "top_k": cfg.k, "routing": cfg.routing, "block_size": 128,
                   "launch": "one CUDA-graph replay per step (4 kernels)",
                   "l2": "before every step 256 MiB are written and then read back, so L2 starts cold and clean (a "
                         "write alone leaves 126 MB of dirty lines that the step would have to write back: "
                         "ms_per_step_dirty_l2); the 1.07 GB of expert weights also exceed L2",
                   "ms_per_step_dirty_l2": ms_per_step_dirty_l2,
                   "frac_of_bf16_peak": value / bf16_tflops},
        "clocks": clocks.summary(),
        "e2e": {"value": cfg.useful_flops / (e2e_ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": e2e_ms_per_step, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "steps pipelined over three streams (copy in, layer as a CUDA-graph replay, copy out), two buffer "
                       "sets; every step's H2D and D2H copies are inside the timed region",
                "single_step_latency_ms": e2e_latency_ms},
        "gpu_launches": 4 * args.steps,
        "roofline": roofline,
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, layer)
    if cfg.name == "fine_grained" and not args.no_scaling_reference:
        # The multi-GPU runs use the expert-parallel workload (E=128, D=F=2048); its one-GPU value is
        # what their per-GPU throughput should be compared with, so it rides along on this line.
        del dev, layer, graph, graph_out, out, h, y, topo
        torch.cuda.empty_cache()
        ep_cfg = CONFIGS["expert_parallel"]
        ep_dev = make_layer(ep_cfg, seed=0).to(device)
        ep_args = (ep_dev.x, ep_dev.expert_idx, ep_dev.expert_weight, ep_dev.w1, ep_dev.w2)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            moe_forward(*ep_args)
        torch.cuda.current_stream().wait_stream(side)
        ep_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(ep_graph):
            ep_out = moe_forward(*ep_args)
        ep_steps = min(args.steps, 50)
        ep_ms = statistics.mean(time_each_ms(ep_graph.replay, flush, warmup=args.warmup, iters=ep_steps))
        line["expert_parallel_1gpu"] = {
            "value": ep_cfg.useful_flops / (ep_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ep_ms, "steps": ep_steps,
            "workload": ep_cfg.name, "how": "the plain layer (all 128 experts on this GPU, no exchange), one graph replay per step",
        }
        del ep_graph, ep_out, ep_dev, ep_args
    print(json.dumps(line))


def run_profile(args: argparse.Namespace) -> None:
    """Three eager layer calls and nothing else: the command to put under ncu."""
    from sparsebench_b200 import moe_forward

    cfg = CONFIGS[args.workload or "fine_grained"]
    torch.cuda.set_device(0)
    dev = make_layer(cfg, seed=0).to("cuda:0")
    for _ in range(3):
        moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    torch.cuda.synchronize()
    print(json.dumps({"profile": cfg.name, "layer_calls": 3}))


def run_expert_parallel(args: argparse.Namespace) -> None:
    from sparsebench_b200 import ep_bench

    ep_bench.run(args, METRIC, measured_peaks(), ClockSampler)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--workload", default=None, choices=sorted(CONFIGS))
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-scaling-reference", action="store_true",
                        help="skip the one-GPU run of the expert-parallel workload that rides along at N=1")
    parser.add_argument("--ep-capacity-factor", type=float, default=3.0,
                        help="expert-parallel exchange rows per rank pair, as a multiple of the even share T*k/N")
    parser.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                        help="expert-parallel exchange: rows stored into peer memory by our kernels, or NCCL all-to-all")
    parser.add_argument("--ep-unfused-return", action="store_true",
                        help="N > 1, peer exchange: DSD writes y and a second kernel pushes it (default: the DSD "
                             "epilogue stores the rows into the source ranks' buffers)")
    parser.add_argument("--ep-micro-batches", type=int, default=0,
                        help="N > 1, peer exchange: cut each step into this many pipelined micro-batches "
                             "(0 = the default for this N)")
    parser.add_argument("--profile", action="store_true", help="run 3 eager layer calls and exit (for ncu)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile:
        run_profile(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    elif args.gpus == 1 and "RANK" not in os.environ:
        run_single_gpu(args)
    else:
        run_expert_parallel(args)


if __name__ == "__main__":
    main()
