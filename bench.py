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
             HBM copy bandwidth (MEASURED_PEAKS.json next to this file, else the stated fallback)
  cpu_baseline  the reference's fp32 CPU implementation of the same layer timed on this machine's
             host cores; its output doubles as the parity check of the GPU result (`parity`)
  other_workloads / expert_parallel_1gpu / library_baselines   the other single-GPU configurations,
             the one-GPU value of the multi-GPU workload, and stock-PyTorch pipelines of the same layer

`config` names the workload only and is identical in both arms; `method` says how it was run.
--impl reference times only the CPU implementation and prints its own line.
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
# Used only if MEASURED_PEAKS.json is absent: an earlier copy-bandwidth / cuBLAS bf16 measurement on B200.
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from profiler captures: a tracked
# table keyed by workload and kernel, each entry with the fingerprint of the kernel sources it was taken on.
TRAFFIC_TABLE = ROOT / "profiles" / "dram_traffic.json"
KERNEL_SOURCES = ["bsr_gemm.cuh", "ptx_sm100.cuh", "sdd.cu", "dsd.cu"]


def kernel_source_fingerprint() -> str:
    import hashlib

    digest = hashlib.sha256()
    for name in KERNEL_SOURCES:
        digest.update((ROOT / "sparsebench_b200" / "csrc" / name).read_bytes())
    return digest.hexdigest()[:16]


def profiled_traffic(workload: str, kernel: str) -> tuple[float | None, str]:
    """(bytes per launch or None, where it comes from / why it is missing)."""
    if not TRAFFIC_TABLE.exists():
        return None, "no profiler capture table"
    for entry in json.loads(TRAFFIC_TABLE.read_text()).get("entries", []):
        if entry.get("workload") == workload and entry.get("kernel") == kernel:
            if entry.get("kernel_sources_sha16") != kernel_source_fingerprint():
                return None, f"stale: captured at {entry.get('commit')} on other kernel sources ({entry.get('summary')})"
            return float(entry["dram_bytes_per_launch"]), f"profiler capture at {entry.get('commit')}: {entry.get('summary')}"
    return None, "no profiler capture of this kernel on this workload"


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
    """ms per step of `forward` fed from pinned HOST buffers when consecutive steps overlap the way a serving loop
    runs them: while step i computes, step i+1's inputs are copied in and step i-1's result is copied out. Two sets
    of device buffers; one CUDA graph per set whose three branches are exactly those three things (the copy-in of
    the OTHER set, this set's layer, the copy-out of the other set's result), so a step is ONE graph launch and the
    host enqueues nothing else. Every step's host->device and device->host copies are inside the timed region; the
    expert weights (far larger than L2) are re-streamed from HBM by every step."""
    host_x, host_idx, host_w = host_inputs
    device = weights[0].device
    main, side_in, side_out = (torch.cuda.Stream(device) for _ in range(3))
    sets = []
    for _ in range(2):
        sets.append({
            "x": torch.empty(host_x.shape, dtype=host_x.dtype, device=device),
            "idx": torch.empty(host_idx.shape, dtype=host_idx.dtype, device=device),
            "w": torch.empty(host_w.shape, dtype=host_w.dtype, device=device),
            "result": torch.empty(host_x.shape, dtype=host_x.dtype, device=device),
            "host_out": torch.empty(host_x.shape, dtype=host_x.dtype).pin_memory(),
        })
    for b in sets:
        b["x"].copy_(host_x)
        b["idx"].copy_(host_idx)
        b["w"].copy_(host_w)
    torch.cuda.synchronize(device)
    with torch.cuda.stream(main):
        forward(sets[0]["x"], sets[0]["idx"], sets[0]["w"], *weights)  # one-time set-up outside the captures
    torch.cuda.synchronize(device)
    graphs = []
    for p in range(2):
        mine, other = sets[p], sets[1 - p]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=main):
            side_in.wait_stream(main)
            side_out.wait_stream(main)
            with torch.cuda.stream(side_in):    # the next step's inputs
                other["x"].copy_(host_x, non_blocking=True)
                other["idx"].copy_(host_idx, non_blocking=True)
                other["w"].copy_(host_w, non_blocking=True)
            with torch.cuda.stream(side_out):   # the previous step's result
                other["host_out"].copy_(other["result"], non_blocking=True)
            mine["result"].copy_(forward(mine["x"], mine["idx"], mine["w"], *weights))  # this step's layer
            main.wait_stream(side_in)
            main.wait_stream(side_out)
        graphs.append(graph)

    def run(n: int) -> None:
        with torch.cuda.stream(main):
            for i in range(n):
                graphs[i % 2].replay()

    torch.cuda.synchronize(device)
    run(max(warmup, 4))
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(main)
    run(steps)
    end.record(main)
    torch.cuda.synchronize(device)
    return start.elapsed_time(end) / steps


def workload_config(cfg: LayerConfig) -> dict:
    """The `config` object of the JSON line: the workload only, identical in both arms."""
    return {"workload": cfg.name, "tokens": cfg.num_tokens, "d_model": cfg.d_model, "ffn_dim": cfg.ffn_dim,
            "experts": cfg.num_experts, "top_k": cfg.k, "routing": cfg.routing, "block_size": 128}


def reference_cpu_layer():
    """(moe_reference, kind): the reference's own CPU implementation (its sparsebench/reference.py, loaded
    unmodified from the copy under baseline/_ref through the `sparsebench` import name) when that copy is
    present, kind "reference"; otherwise the oracle's restatement of it, kind "port"."""
    try:
        import sparsebench

        if sparsebench.reference_py_dir() is not None:
            from sparsebench.reference import moe_reference

            return moe_reference, "reference"
    except Exception:  # noqa: BLE001 - fall through to the port
        pass
    from oracle import moe as oracle_moe

    return oracle_moe.moe_reference, "port"


def cpu_baseline(cfg: LayerConfig, layer, gpu_out: torch.Tensor | None, budget_s: float = 20.0) -> tuple[dict, dict]:
    """The reference's fp32 CPU layer on this machine's host cores: (cpu_baseline, parity). Its output is
    also the check of the GPU result: every row of `gpu_out` against it, rtol = atol = 2e-2."""
    moe_reference, kind = reference_cpu_layer()
    x, w = layer.x.float(), layer.expert_weight.float()
    w1, w2 = layer.w1.float(), layer.w2.float()
    times = []
    started = time.perf_counter()
    expected = None
    for i in range(7):
        t0 = time.perf_counter()
        expected = moe_reference(x, layer.expert_idx, w, w1, w2)
        dt = time.perf_counter() - t0
        if i >= 2:
            times.append(dt)
        if time.perf_counter() - started > budget_s and len(times) >= 1:
            break
    med = statistics.median(times)
    baseline = {
        "value": cfg.useful_flops / med / 1e12,
        "unit": "TFLOP/s",
        "ms_per_step": med * 1e3,
        "cores": torch.get_num_threads(),
        "host_cpus": os.cpu_count(),
        "kind": kind,
        "sample": f"whole {cfg.name} layer in fp32, median of {len(times)} runs after 2 warm-up runs",
    }
    parity = {"ok": None, "reason": "no GPU output given"}
    if gpu_out is not None:
        got = gpu_out.float().cpu()
        err = (got - expected).abs()
        parity = {"rows_checked": int(got.shape[0]), "max_abs_err": float(err.max()),
                  "ok": bool((err <= 2e-2 + 2e-2 * expected.abs()).all()),
                  "against": f"the reference's fp32 CPU layer ({kind}) on the same bf16 inputs, rtol = atol = 2e-2"}
    return baseline, parity


def run_reference_arm(args: argparse.Namespace) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = CONFIGS[args.workload or ("fine_grained" if args.gpus == 1 else "expert_parallel")]
    if args.gpus > 1:
        import bench_ep

        config = bench_ep.workload_config(cfg, args.gpus)
        # the CPU arm computes (a sample of) the global batch of all ranks' tokens
        cfg = LayerConfig(cfg.name, cfg.num_tokens * args.gpus, cfg.d_model, cfg.ffn_dim, cfg.num_experts, cfg.routing)
    else:
        config = workload_config(cfg)
    moe_reference, kind = reference_cpu_layer()

    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm is alone on the host, so it takes
    # every core the process may run on.
    torch.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    layer = make_layer(cfg, seed=0)
    x, w = layer.x.float(), layer.expert_weight.float()
    w1, w2 = layer.w1.float(), layer.w2.float()
    # A step here is a bounded sample: the first `sample_tokens` tokens of the batch through the whole
    # layer, halved until steps + warmup fit in about four minutes on the host cores.
    sample_tokens = min(cfg.num_tokens, 4096)
    steps, warmup = args.steps, args.warmup
    while True:
        xs, idx, ws = x[:sample_tokens], layer.expert_idx[:sample_tokens], w[:sample_tokens]
        t0 = time.perf_counter()
        moe_reference(xs, idx, ws, w1, w2)
        if (time.perf_counter() - t0) * (steps + warmup) <= 240.0 or sample_tokens <= 64:
            break
        sample_tokens //= 2
    for _ in range(max(0, warmup - 1)):
        moe_reference(xs, idx, ws, w1, w2)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        moe_reference(xs, idx, ws, w1, w2)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    flops = 4 * sample_tokens * cfg.k * cfg.d_model * cfg.ffn_dim
    value = flops / sec / 1e12
    sample = (f"{sample_tokens} of {cfg.num_tokens} tokens through the whole fp32 layer per step, median of {steps} "
              f"steps after {warmup} warm-up steps")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def live_rows(expert_idx: torch.Tensor, num_experts: int, granule: int = 128) -> int:
    """Rows of the layout after rounding every expert's copies up to `granule`: 128 is what the tensor
    cores execute (whole row blocks), 32 what SDD stores and DSD loads and stores in the layer (groups
    of 32 rows that are all padding are skipped)."""
    counts = torch.bincount(expert_idx.reshape(-1), minlength=num_experts)
    return int(((counts + granule - 1) // granule * granule).sum())


def capture_layer(dev):
    """(graph, graph_out, eager_out) of moe_forward over the fixed device tensors of `dev`."""
    from sparsebench_b200 import moe_forward

    args = (dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    out = moe_forward(*args)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        moe_forward(*args)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_out = moe_forward(*args)
    torch.cuda.synchronize()
    return graph, graph_out, out


def require_clean_status(device: torch.device, when: str) -> None:
    from sparsebench_b200 import _C

    status = int(_C.device_status(device).item())
    if status != 0:
        raise SystemExit(f"{when}: device status word is {status}: a bounded device-side wait of a matmul kernel expired")


def stage_roofline(cfg: LayerConfig, layer, dev, flush, iters: int, peaks: tuple[float, float, str]) -> dict:
    """Each kernel's time in its place in the layer and the roofline of the slower matmul."""
    from sparsebench_b200 import route_device
    from sparsebench_b200.spmm import combine, dsd, sdd
    from sparsebench_b200.timing import marginal_stage_times_ms

    hbm_gbs, bf16_tflops, peak_kind = peaks
    w2_cat = dev.w2.view(cfg.num_experts * cfg.ffn_dim, cfg.d_model)

    def stage_route(state: dict) -> None:
        state["topo"] = route_device(dev.expert_idx, cfg.num_experts, cfg.ffn_dim, 128)

    def stage_sdd(state: dict) -> None:
        state["h"] = sdd(dev.x, dev.w1, state["topo"], skip_padding_rows=True, layout_from_routing=True)

    def stage_dsd(state: dict) -> None:
        state["y"] = dsd(state["h"], w2_cat, state["topo"], version=5, skip_padding_rows=True, layout_from_routing=True)

    def stage_combine(state: dict) -> None:
        state["out"] = combine(state["y"], dev.expert_weight, state["topo"])

    stage_ms = marginal_stage_times_ms([("routing", stage_route), ("sdd", stage_sdd), ("dsd", stage_dsd),
                                        ("combine", stage_combine)], flush, 3, iters)
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
    dominant = max(("sdd", "dsd"), key=lambda name: stage_ms[name])
    t_dom = stage_ms[dominant] * 1e-3
    hbm_time = stage_bytes[dominant] / (hbm_gbs * 1e9)
    exec_flops = 2 * rows * cfg.d_model * cfg.ffn_dim  # one matmul, padding rows included
    if hbm_time >= exec_flops / (bf16_tflops * 1e12):
        achieved = stage_bytes[dominant] / t_dom / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs}
    else:
        achieved = exec_flops / t_dom / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": bf16_tflops, "unit": "TFLOP/s",
                    "frac": achieved / bf16_tflops}
    traffic, traffic_source = profiled_traffic(cfg.name, dominant)
    roofline.update({
        "kernel": f"bsr_gemm_kernel<{dominant}>",
        "peak_source": f"{peak_kind} (MEASURED_PEAKS.json)" if peak_kind == "measured" else "fallback",
        "launch_ms": stage_ms[dominant], "algorithmic_bytes": stage_bytes[dominant], "live_rows": rows,
        "rows_moved": rows_moved, "traffic": traffic, "traffic_source": traffic_source,
        "stages_ms": stage_ms,
        "stages_timing": "each kernel in its place in the layer: CUDA-graph replays of the first j stages (each closed by "
                         "the same one-element kernel), CUDA events around every replay, L2 flushed before it, stage j = "
                         "prefix j - prefix j-1",
        "stages_frac_of_hbm_peak": {name: stage_bytes[name] / (stage_ms[name] * 1e-3) / 1e9 / hbm_gbs for name in stage_bytes},
        "stages_executed_tflops": {name: exec_flops / (stage_ms[name] * 1e-3) / 1e12 for name in stage_flops},
        "stages_useful_tflops": {name: stage_flops[name] / (stage_ms[name] * 1e-3) / 1e12 for name in stage_flops},
    })
    return roofline


def measure_other_workload(name: str, args: argparse.Namespace, device: torch.device, flush: torch.Tensor,
                           peaks: tuple[float, float, str], with_stages: bool = True) -> dict:
    """One of the other single-GPU configurations, measured like the headline one (graph replays, L2 flushed,
    clocks sampled during its own timed region), without the end-to-end and CPU legs."""
    from sparsebench_b200.timing import time_each_ms

    cfg = CONFIGS[name]
    layer = make_layer(cfg, seed=0)
    dev = layer.to(device)
    graph, graph_out, out = capture_layer(dev)
    steps = min(args.steps, 50)
    with ClockSampler(0) as clocks:
        torch.cuda.synchronize()
        ms = statistics.mean(time_each_ms(graph.replay, flush, warmup=args.warmup, iters=steps))
        torch.cuda.synchronize()
    if not torch.equal(graph_out, out):
        raise SystemExit(f"{name}: graph replay and eager launch disagree")
    require_clean_status(device, f"{name}, after the timed steps")
    row = {"value": cfg.useful_flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
           "config": workload_config(cfg), "clocks": clocks.summary(),
           "frac_of_bf16_peak": cfg.useful_flops / (ms * 1e-3) / 1e12 / peaks[1]}
    if with_stages:
        row["roofline"] = stage_roofline(cfg, layer, dev, flush, max(5, min(args.steps, 20)), peaks)
    del graph, graph_out, out, dev, layer
    torch.cuda.empty_cache()
    return row


def reference_gpu_row(workload: str) -> dict:
    """The reference's own CUDA kernels (compiled for sm_100 by oracle/build_ref_ext.py) on this GPU, as a
    comparison row measured in a child process, so that this process never loads them."""
    import subprocess

    try:
        proc = subprocess.run([sys.executable, str(ROOT / "bench_baselines.py"), "--reference-gpu", workload],
                              capture_output=True, text=True, timeout=300, cwd=ROOT)
        for text in reversed(proc.stdout.splitlines()):
            if text.startswith("{"):
                return json.loads(text)
        return {"unavailable": f"no result (exit code {proc.returncode}): {proc.stderr[-200:]}"}
    except Exception as exc:  # noqa: BLE001 - a comparison row, never fatal
        return {"unavailable": repr(exc)[:200]}


def run_single_gpu(args: argparse.Namespace) -> None:
    from sparsebench_b200 import moe_forward
    from sparsebench_b200.timing import l2_flush_buffer, time_each_ms

    cfg = CONFIGS[args.workload or "fine_grained"]
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    layer = make_layer(cfg, seed=0)
    dev = layer.to(device)
    flush = l2_flush_buffer(device)
    peaks = measured_peaks()
    hbm_gbs, bf16_tflops, peak_kind = peaks

    # ---- correctness gate before timing anything: every output row against the reference's CPU layer ------
    graph, graph_out, out = capture_layer(dev)
    require_clean_status(device, "first layer call")
    baseline, parity = (None, {"ok": None, "reason": "--no-cpu-baseline"})
    if not args.no_cpu_baseline:
        baseline, parity = cpu_baseline(cfg, layer, out)
        if not parity["ok"]:
            raise SystemExit(f"the layer's output differs from the reference's CPU layer: {parity}")

    # ---- value: graph replay, inputs resident in HBM ------------------------------------------------
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
        raise SystemExit("graph replay and eager launch disagree")
    require_clean_status(device, "after the timed steps")

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
    require_clean_status(device, "after the end-to-end steps")
    h2d = host_x.numel() * host_x.element_size() + host_idx.numel() * host_idx.element_size() + \
        host_w.numel() * host_w.element_size()
    d2h = host_out.numel() * host_out.element_size()

    roofline = stage_roofline(cfg, layer, dev, flush, max(5, min(args.steps, 50)), peaks)

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(cfg),
        "method": {"launch": "one CUDA-graph replay per step (4 kernels)",
                   "l2": "before every step 256 MiB are written and then read back, so L2 starts cold and clean (a "
                         "write alone leaves 126 MB of dirty lines that the step would have to write back: "
                         "ms_per_step_dirty_l2); the expert weights also exceed L2",
                   "ms_per_step_dirty_l2": ms_per_step_dirty_l2,
                   "frac_of_bf16_peak": value / bf16_tflops},
        "parity": parity,
        "clocks": clocks.summary(),
        "e2e": {"value": cfg.useful_flops / (e2e_ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": e2e_ms_per_step, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "steps pipelined: one CUDA-graph launch per step whose three branches are the next step's H2D copy, "
                       "this step's layer and the previous step's D2H copy (two buffer sets); every step's copies are "
                       "inside the timed region",
                "single_step_latency_ms": e2e_latency_ms},
        "gpu_launches": 4 * args.steps,
        "roofline": roofline,
    }
    if baseline is not None:
        line["cpu_baseline"] = baseline
    if cfg.name == "fine_grained" and not args.no_library_baselines:
        import bench_baselines

        line["library_baselines"] = {
            "what": "the same layer with stock PyTorch kernels on this GPU (eager calls, CUDA events, L2 flushed); "
                    "context, not the product path",
            "this_library_eager_ms": statistics.median(time_each_ms(
                lambda: moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2), flush, 3, 20)),
            "pipelines": bench_baselines.measure(cfg, dev, flush, out, iters=20),
        }
    del graph, graph_out, out, dev
    torch.cuda.empty_cache()
    if cfg.name == "fine_grained" and not args.no_library_baselines:
        line["reference_gpu_kernels"] = reference_gpu_row(cfg.name)
    if cfg.name == "fine_grained" and not args.no_other_workloads:
        # The other single-GPU configurations, each with its own clock record (the Mixtral-like one is the
        # shape that runs into the power cap).
        line["other_workloads"] = {name: measure_other_workload(name, args, device, flush, peaks)
                                   for name in ("fine_grained_zipf", "mixtral_like")}
    if cfg.name == "fine_grained" and not args.no_scaling_reference:
        # The multi-GPU runs use the expert-parallel workload (E=128, D=F=2048); its one-GPU value is
        # what their per-GPU throughput should be compared with, so it rides along on this line.
        row = measure_other_workload("expert_parallel", args, device, flush, peaks, with_stages=False)
        row["how"] = "the plain layer (all 128 experts on this GPU, no exchange), one graph replay per step"
        row["workload"] = "expert_parallel"
        line["expert_parallel_1gpu"] = row
    print(json.dumps(line))


def run_profile(args: argparse.Namespace) -> None:
    """Three eager layer calls and nothing else: the command to put under ncu. With --profile-front-ends the
    three calls go through the router, the token-rounding and the assignment-list front ends instead, so that
    their small kernels show up too."""
    from sparsebench_b200 import moe_forward, moe_forward_from_logits, moe_forward_rounded, route

    cfg = CONFIGS[args.workload or "fine_grained"]
    torch.cuda.set_device(0)
    dev = make_layer(cfg, seed=0).to("cuda:0")
    if args.profile_front_ends:
        g = torch.Generator().manual_seed(0)
        logits = torch.randn(cfg.num_tokens, cfg.num_experts, generator=g).to("cuda:0")
        scores = torch.softmax(logits, dim=-1)
        for _ in range(3):
            moe_forward_from_logits(dev.x, logits, dev.w1, dev.w2, k=cfg.k, one_launch_routing=True)  # router inside routing
            route(logits, cfg.k)                                             # the router as a kernel of its own
            moe_forward_rounded(dev.x, scores, dev.w1, dev.w2, k=cfg.k)      # rounding, assignment list, scatter-add combine
        torch.cuda.synchronize()
        print(json.dumps({"profile": cfg.name, "front_end_rounds": 3}))
        return
    for _ in range(3):
        moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    torch.cuda.synchronize()
    print(json.dumps({"profile": cfg.name, "layer_calls": 3}))


def run_expert_parallel(args: argparse.Namespace) -> None:
    import bench_ep

    bench_ep.run(args, METRIC, measured_peaks(), ClockSampler)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--workload", default=None, choices=sorted(CONFIGS))
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-other-workloads", action="store_true",
                        help="skip the fine_grained_zipf and mixtral_like runs that ride along at N=1")
    parser.add_argument("--no-library-baselines", action="store_true",
                        help="skip the stock-PyTorch pipelines (torch._grouped_mm, per-expert loop, padded bmm) at N=1")
    parser.add_argument("--no-scaling-reference", action="store_true",
                        help="skip the one-GPU run of the expert-parallel workload that rides along at N=1")
    parser.add_argument("--ep-capacity-factor", type=float, default=3.0,
                        help="expert-parallel exchange rows per rank pair, as a multiple of the even share T*k/N")
    parser.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                        help="expert-parallel exchange: rows stored into peer memory by our kernels, or NCCL all-to-all")
    parser.add_argument("--ep-unfused-return", action="store_true",
                        help="N > 1, peer exchange: DSD writes y and a second kernel pushes it (default: the DSD "
                             "epilogue stores the rows into the source ranks' buffers)")
    parser.add_argument("--ep-dispatch", default="auto", choices=["auto", "beside", "overlapped", "separate"],
                        help="N > 1, peer exchange: 'separate' pushes all rows and waits for every rank before the "
                             "owner's routing; 'beside' runs the push kernel on a second stream beside the owner's SDD "
                             "kernel, whose tiles wait for the segments they need; 'overlapped' lets extra warps of "
                             "that SDD kernel push the rows; 'auto' takes the measured default for this N")
    parser.add_argument("--ep-unfused-dispatch", action="store_true", help="same as --ep-dispatch separate")
    parser.add_argument("--no-nccl-context", action="store_true",
                        help="N > 1: skip the few extra steps with NCCL all-to-all collectives as the exchange")
    parser.add_argument("--ep-micro-batches", type=int, default=0,
                        help="N > 1, peer exchange: cut each step into this many pipelined micro-batches "
                             "(0 = the default for this N)")
    parser.add_argument("--ep-micro-split", default="",
                        help="N > 1, peer exchange: shares of the micro-batches, e.g. 0.25,0.75 (default: equal shares)")
    parser.add_argument("--profile", action="store_true", help="run 3 eager layer calls and exit (for ncu)")
    parser.add_argument("--profile-front-ends", action="store_true",
                        help="with --profile: run the router, token-rounding and assignment-list front ends of the layer")
    parser.add_argument("--profile-ep-owner", action="store_true",
                        help="ONE GPU: rank 0's owner-side kernels of the 8-rank expert-parallel step at full size, "
                             "exchange buffers in local memory, three times, then exit (for ncu)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile_ep_owner:
        import bench_ep

        bench_ep.run_owner_profile(args)
    elif args.profile:
        run_profile(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    elif args.gpus == 1 and "RANK" not in os.environ:
        run_single_gpu(args)
    else:
        run_expert_parallel(args)


if __name__ == "__main__":
    main()
