"""The expert-parallel arm of bench.py: one rank per GPU under torchrun (or a single process for
world size 1). Weak scaling: every rank brings T tokens, the E experts are split over the ranks.

Timing: CUDA events around every step on the launching stream, 256 MiB written and read back before
every step to flush L2, a barrier and a device synchronise on both sides of the timed region, per-rank sums
reduced with MAX. The step is one CUDA-graph replay when the collectives can be captured, else
eager launches (config.launch says which).
"""

from __future__ import annotations

import glob
import json
import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from sparsebench_b200.ep import ExpertParallelMoE  # noqa: E402
from sparsebench_b200.timing import flush_l2, l2_flush_buffer  # noqa: E402
from sparsebench_b200.workloads import CONFIGS, _weights, make_layer  # noqa: E402

NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer-to-peer copy bandwidth of one B200 over NVLink 5; 900 nominal
PARITY_ROWS_PER_RANK = 32

# The form of the peer-exchange step per rank count, as measured on this machine: (dispatch overlapped inside the
# owner's SDD kernel, micro-batches pipelined over streams). Rank counts that are not listed run the plainest form.
DEFAULT_EP_FORM: dict[int, tuple[bool, int]] = {2: (False, 1), 4: (False, 1), 8: (False, 2)}
DEFAULT_MICRO_BATCHES: dict[int, int] = {n: form[1] for n, form in DEFAULT_EP_FORM.items()}
# Unequal shares of the micro-batches where measured to pay (the first part's dispatch is the one nothing hides).
DEFAULT_MICRO_FRACTIONS: dict[int, tuple[float, ...]] = {}


def overlapped_dispatch_wanted(args, world: int) -> bool:
    """--ep-dispatch beside / overlapped / separate, the older --ep-unfused-dispatch, else the table above."""
    choice = getattr(args, "ep_dispatch", "auto")
    if getattr(args, "ep_unfused_dispatch", False) or choice == "separate":
        return False
    if choice in ("overlapped", "beside"):
        return True
    return DEFAULT_EP_FORM.get(world, (False, 1))[0]



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


class PackedStaging:
    """One pinned host buffer per direction and one device staging buffer per buffer set, holding the
    step's inputs back to back (each part 256-byte aligned), so that a step is ONE host->device copy and
    ONE device->host copy instead of one per tensor. Device-side views give the parts their shapes."""

    def __init__(self, tensors: list[torch.Tensor], device: torch.device) -> None:
        self.offsets, total = [], 0
        for t in tensors:
            self.offsets.append(total)
            total += (t.numel() * t.element_size() + 255) // 256 * 256
        self.host = torch.empty(total, dtype=torch.uint8).pin_memory()
        for t, off in zip(tensors, self.offsets):
            nbytes = t.numel() * t.element_size()
            self.host[off:off + nbytes].copy_(t.contiguous().view(-1).view(torch.uint8))
        self.shapes = [(t.shape, t.dtype) for t in tensors]
        self.device, self.total = device, total

    def device_buffer(self) -> torch.Tensor:
        return torch.empty(self.total, dtype=torch.uint8, device=self.device)

    def views(self, buffer: torch.Tensor) -> list[torch.Tensor]:
        out = []
        for off, (shape, dtype) in zip(self.offsets, self.shapes):
            nbytes = int(torch.tensor(shape).prod().item()) * torch.empty(0, dtype=dtype).element_size()
            out.append(buffer[off:off + nbytes].view(dtype).view(shape))
        return out


def _pipelined_e2e_ms(step, result_of, dev_inputs, staging: PackedStaging, warmup: int, steps: int, world: int) -> float:
    """Mean ms per step, max over ranks, of the step fed from pinned HOST buffers when consecutive steps
    overlap the way a serving loop runs them: three streams (copy in, step, copy out) and two sets of
    staging buffers. `step` reads fixed device tensors (a captured graph does), so the compute stream
    first copies the staged inputs into them (device to device, a few us) and the result out into the
    set's staging tensor. Every step's host->device copy (one packed buffer) and device->host copy are
    inside the timed region."""
    device = dev_inputs[0].device
    copy_in, compute, copy_out = (torch.cuda.Stream(device) for _ in range(3))
    sets = []
    for _ in range(2):
        staged = staging.device_buffer()
        sets.append({
            "staged": staged, "in": staging.views(staged),
            "out": torch.empty_like(dev_inputs[0]),
            "host_out": torch.empty(dev_inputs[0].shape, dtype=dev_inputs[0].dtype).pin_memory(),
            "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "copied": torch.cuda.Event(),
        })

    def run(n: int) -> None:
        for i in range(n):
            b = sets[i % 2]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(b["computed"])  # the step that last read this set's inputs is done
                b["staged"].copy_(staging.host, non_blocking=True)
                b["loaded"].record(copy_in)
            with torch.cuda.stream(compute):
                compute.wait_event(b["loaded"])
                compute.wait_event(b["copied"])  # this set's result tensor has been read out
                for fixed, part in zip(dev_inputs, b["in"]):
                    fixed.copy_(part, non_blocking=True)
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


def _cpu_list(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if part:
            first, _, last = part.partition("-")
            cpus.update(range(int(first), int(last or first) + 1))
    return cpus


def bind_to_gpu_numa_node(local: int) -> dict:
    """Restricts THIS process to the CPUs of the NUMA node its GPU hangs off, so that the pinned
    staging buffers it allocates next are placed in that node's memory (first touch) and the copy
    engine does not pull every rank's tokens across the socket interconnect. Reads sysfs only; changes
    nothing outside this process. Returns what it found for the JSON line."""
    info: dict = {"numa_node": None, "bound": False}
    try:
        import pynvml

        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        physical = int(visible.split(",")[local]) if visible and visible.replace(",", "").isdigit() else local
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(physical)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
        info["numa_node"] = node
        nodes = sorted(glob.glob("/sys/devices/system/node/node*/cpulist"))
        info["numa_nodes"] = len(nodes)
        if node >= 0 and len(nodes) > 1:
            cpus = _cpu_list(Path(f"/sys/devices/system/node/node{node}/cpulist").read_text()) & os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                info["bound"], info["cpus"] = True, len(cpus)
    except Exception as exc:  # noqa: BLE001 - placement is an optimisation; say why it was skipped
        info["skipped"] = repr(exc)[:120]
    return info


def host_link_gbs(device: torch.device, world: int) -> dict:
    """Host<->device copy bandwidth of pinned memory with ALL ranks copying at the same time (what the
    end-to-end loop can get at best): per direction, this rank's GB/s reduced to min / sum over ranks."""
    nbytes = 128 * 1024 * 1024
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    host.fill_(1)
    dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
    out = {}
    for name, copy in (("h2d", lambda: dev.copy_(host, non_blocking=True)), ("d2h", lambda: host.copy_(dev, non_blocking=True))):
        copy()
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(4):
            copy()
        end.record()
        end.synchronize()
        mine = torch.tensor([4 * nbytes / (start.elapsed_time(end) * 1e-3) / 1e9], dtype=torch.float64, device=device)
        total, least = mine.clone(), mine.clone()
        if world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            dist.all_reduce(least, op=dist.ReduceOp.MIN)
        out[name] = {"all_ranks_gbs": float(total.item()), "slowest_rank_gbs": float(least.item())}
    # Both directions at once on two streams, as the pipelined end-to-end loop runs them: bytes moved either way per
    # second. The loop cannot be faster than (bytes in + bytes out per step) / this figure.
    dev_out = torch.empty(nbytes, dtype=torch.uint8, device=device)
    host_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    inbound, outbound = torch.cuda.Stream(device), torch.cuda.Stream(device)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    inbound.wait_event(start)
    outbound.wait_event(start)
    for _ in range(4):
        with torch.cuda.stream(inbound):
            dev.copy_(host, non_blocking=True)
        with torch.cuda.stream(outbound):
            host_out.copy_(dev_out, non_blocking=True)
    torch.cuda.current_stream().wait_stream(inbound)
    torch.cuda.current_stream().wait_stream(outbound)
    end.record()
    end.synchronize()
    mine = torch.tensor([8 * nbytes / (start.elapsed_time(end) * 1e-3) / 1e9], dtype=torch.float64, device=device)
    total, least = mine.clone(), mine.clone()
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        dist.all_reduce(least, op=dist.ReduceOp.MIN)
    out["both_directions"] = {"all_ranks_gbs": float(total.item()), "slowest_rank_gbs": float(least.item())}
    return out


def parity_sample(cfg, layer_in, out: torch.Tensor, world: int, rows: int = PARITY_ROWS_PER_RANK) -> dict:
    """The first `rows` output rows of THIS rank against the fp32 CPU oracle (rtol = atol = 2e-2), over
    exactly the experts those tokens use (weights regenerated from their per-expert seeds); the verdicts
    of all ranks are reduced. The oracle is only the checker here; nothing timed touches it."""
    from oracle import moe as oracle_moe

    idx = layer_in.expert_idx[:rows]
    used = sorted(set(idx.reshape(-1).tolist()))
    position = {e: i for i, e in enumerate(used)}
    local_idx = torch.tensor([[position[e] for e in row] for row in idx.tolist()])
    w1 = _weights(0, used, cfg.d_model, cfg.ffn_dim, 0, torch.bfloat16).float()
    w2 = _weights(1, used, cfg.ffn_dim, cfg.d_model, 0, torch.bfloat16).float()
    expected = oracle_moe.moe_reference(layer_in.x[:rows].float(), local_idx, layer_in.expert_weight[:rows].float(), w1, w2)
    got = out[:rows].float().cpu()
    err = (got - expected).abs()
    ok = bool((err <= 2e-2 + 2e-2 * expected.abs()).all())
    verdict = torch.tensor([float(ok), -float(err.max())], dtype=torch.float64, device=out.device)
    if world > 1:
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    return {"rows_checked": rows * world, "max_abs_err": -float(verdict[1].item()), "ok": bool(verdict[0].item() == 1.0),
            "against": "fp32 CPU oracle of the layer on each rank's first rows, rtol = atol = 2e-2"}


def check_status(moe, device: torch.device, world: int, when: str) -> None:
    """Raises if any rank's expert-parallel status word or matmul status word is set. Syncs."""
    from sparsebench_b200 import _C

    words = torch.cat([moe.status.to(torch.int32), _C.device_status(device).to(torch.int32)]).clone()
    if world > 1:
        gathered = [torch.empty_like(words) for _ in range(world)]
        dist.all_gather(gathered, words)
    else:
        gathered = [words]
    problems = []
    for r, w in enumerate(gathered):
        ep, gemm = int(w[0].item()), int(w[1].item())
        if ep & 1:
            problems.append(f"rank {r}: the exchange overflowed its capacity (rows were dropped)")
        if ep & 2:
            problems.append(f"rank {r}: a device-side barrier timed out waiting for a peer rank")
        if ep & ~3:
            problems.append(f"rank {r}: expert-parallel status word {ep}")
        if gemm:
            problems.append(f"rank {r}: a bounded wait inside a matmul kernel expired (status {gemm})")
    if problems:
        raise SystemExit(f"{when}: " + "; ".join(problems))


class LocalExchange:
    """The exchange buffers of `ranks` virtual ranks, all in ONE GPU's memory, with the peer tables pointing at
    them: lets a single GPU run one rank's kernels of the multi-GPU step at full size (profilers never wrap a
    multi-rank command). of(r) has the attribute names of sparsebench_b200.ep.PeerExchange."""

    def __init__(self, ranks: int, capacity: int, d_model: int, experts_local: int, device: torch.device) -> None:
        segments = (capacity + 255) // 256  # arrival flags per rank pair (sb_ep_dispatch_segments)
        self.recv = torch.zeros(ranks, ranks * capacity, d_model, dtype=torch.bfloat16, device=device)
        self.ret = torch.zeros(ranks, ranks * capacity, d_model, dtype=torch.bfloat16, device=device)
        self.counts = torch.zeros(ranks, ranks, experts_local, dtype=torch.int32, device=device)
        self.pad = torch.zeros(ranks, ranks, dtype=torch.int32, device=device)
        self.flags = torch.zeros(ranks, ranks * segments, dtype=torch.int32, device=device)
        self.epoch = [torch.zeros(1, dtype=torch.int32, device=device) for _ in range(ranks)]
        self.done = [torch.zeros(ranks * segments, dtype=torch.int32, device=device) for _ in range(ranks)]

        def table(t: torch.Tensor) -> torch.Tensor:
            return torch.tensor([t[r].data_ptr() for r in range(ranks)], dtype=torch.int64, device=device)

        self.peer_recv, self.peer_ret = table(self.recv), table(self.ret)
        self.peer_counts, self.peer_pads, self.peer_flags = table(self.counts), table(self.pad), table(self.flags)

    def of(self, rank: int):
        import types

        return types.SimpleNamespace(
            recv=self.recv[rank], ret=self.ret[rank], counts=self.counts[rank], pad=self.pad[rank], flags=self.flags[rank],
            epoch=self.epoch[rank], done=self.done[rank], peer_recv=self.peer_recv, peer_ret=self.peer_ret,
            peer_counts=self.peer_counts, peer_pads=self.peer_pads, peer_flags=self.peer_flags)


def run_owner_profile(args) -> None:
    """ONE GPU, the owner-side kernels of rank 0 of the 8-rank expert-parallel step at full size, three times:
    the other seven ranks' rows are pushed by the stand-alone push kernel first (one virtual rank at a time,
    nothing waits for a concurrent launch), then rank 0's owner layout, SDD with its own pushes inside, and DSD
    with the return stores inside. The command to put under a profiler for those kernels."""
    from sparsebench_b200 import _C
    from sparsebench_b200.routing import DeviceTopology

    ranks = 8
    cfg = CONFIGS[args.workload or "expert_parallel"]
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    experts_local = cfg.num_experts // ranks
    n_copies = cfg.num_tokens * cfg.k
    capacity = int(math.ceil(3.0 * n_copies / ranks / 128.0)) * 128  # keeps the buffers near 1 GB in total
    ex = LocalExchange(ranks, capacity, cfg.d_model, experts_local, device)
    mine = make_layer(cfg, seed=0, token_seed=0, experts=range(experts_local)).to(device)
    sorts, starts, xs = [], [], []
    for rank in range(ranks):
        tokens = make_layer(cfg, seed=0, token_seed=rank, experts=range(0)).to(device)
        counts, offsets, sorted_token, _, _ = _C.sort_copies_cuda(tokens.expert_idx, cfg.num_experts)
        ex.epoch[rank].fill_(1)
        _C.ep_push_counts(counts, ex.peer_counts, rank, experts_local)
        starts.append(offsets)
        sorts.append(sorted_token)
        xs.append(tokens.x)
    w2_cat = mine.w2.view(experts_local * cfg.ffn_dim, cfg.d_model)
    view = ex.of(0)
    for step in range(3):
        for rank in range(ranks):
            ex.epoch[rank].fill_(step + 1)
        for rank in range(1, ranks):
            r = ex.of(rank)
            _C.ep_push_rows_flagged(xs[rank], sorts[rank], starts[rank], ex.peer_recv, ex.peer_flags, r.done, r.epoch, rank,
                                    experts_local, capacity)
        torch.cuda.synchronize()
        *layout, order = _C.ep_owner_layout(view.counts, capacity, cfg.ffn_dim, arrival_order=True)
        topo = DeviceTopology(128, experts_local, cfg.ffn_dim // 128, *layout)
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda._sleep(2_000_000)  # about a millisecond of GPU time: the launches below queue up behind it
        marks[0].record()
        h = _C.ep_sdd_dispatch(view.recv, mine.w1, topo.row_token, topo.row_block_expert, topo.row_offsets,
                               topo.col_indices.numel(), xs[0], sorts[0], starts[0],
                               order, ex.peer_recv, ex.peer_flags,
                               view.flags, view.done, view.epoch, 0, capacity)
        marks[1].record()
        _C.ep_dsd_push(h, w2_cat, topo.row_offsets, topo.col_indices, topo.row_token, ex.peer_ret, 0, capacity)
        marks[2].record()
        _C.sdd_cuda(view.recv, mine.w1, topo.row_token, topo.row_block_expert, topo.row_offsets,
                    topo.col_indices.numel(), True, True, topo.padded_offsets)
        marks.append(torch.cuda.Event(enable_timing=True))
        marks[3].record()
        torch.cuda.synchronize()
        kernel_ms = {"sdd_with_pushes": marks[0].elapsed_time(marks[1]), "dsd_with_return": marks[1].elapsed_time(marks[2]),
                     "plain_sdd_same_layout": marks[2].elapsed_time(marks[3])}
    status = int(_C.device_status(device).item())
    rows = int(topo.padded_offsets[-1].item())
    print(json.dumps({"profile": "expert-parallel owner, rank 0 of 8 on one GPU", "steps": 3, "padded_rows": rows,
                      "received_rows": int(view.counts.sum().item()), "capacity_rows_per_pair": capacity,
                      "last_step_kernel_ms": kernel_ms, "device_status": status}))
    if status != 0:
        raise SystemExit("a bounded device-side wait expired")


def workload_config(cfg, world: int) -> dict:
    """The `config` object of the JSON line: the workload only, identical for this arm and the reference arm."""
    return {"workload": cfg.name, "tokens_per_gpu": cfg.num_tokens, "d_model": cfg.d_model, "ffn_dim": cfg.ffn_dim,
            "experts": cfg.num_experts, "top_k": cfg.k, "routing": cfg.routing, "gpus": world}


def run(args, metric: str, peaks: tuple[float, float, str], clock_sampler_cls) -> None:
    """Measures the expert-parallel step on every rank; rank 0 prints the JSON line."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    placement = bind_to_gpu_numa_node(local) if world > 1 else {"bound": False}
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    line = measure(args, metric, peaks, clock_sampler_cls, world, rank, local)
    line.setdefault("e2e", {})["host_placement"] = placement
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
    # Shares of the micro-batches ("0.25,0.75"); empty = the default for this rank count, else equal shares.
    split = getattr(args, "ep_micro_split", "") or ""
    micro_fractions = tuple(float(f) for f in split.split(",")) if split else None
    if micro_fractions is None and not getattr(args, "ep_micro_batches", 0):
        micro_fractions = DEFAULT_MICRO_FRACTIONS.get(world)
    if micro_fractions is not None:
        micro_batches = len(micro_fractions)
    moe = None
    if exchange == "peer":
        # Rows stored straight into the owner's memory: only real rows travel, so the capacity can be
        # the exact worst case. If the buffers cannot be mapped on this machine every rank falls back.
        try:
            moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=n_copies, exchange="peer",
                                    fuse_return=not getattr(args, "ep_unfused_return", False),
                                    fuse_dispatch=overlapped_dispatch_wanted(args, world),
                                    push_beside=getattr(args, "ep_dispatch", "auto") != "overlapped",
                                    micro_fractions=micro_fractions,
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

    def first_step_ok(layer) -> tuple[torch.Tensor, dict]:
        result = layer(dev.x, dev.expert_idx, dev.expert_weight)
        torch.cuda.synchronize()
        check_status(layer, device, world, "first step")
        # ---- parity gate before anything is timed ----------------------------------------------------
        verdict = parity_sample(cfg, layer_in, result, world)
        if not verdict["ok"]:
            raise SystemExit(f"expert-parallel output differs from the oracle: {verdict}")
        return result, verdict

    fallback_note = None
    try:
        out, parity = first_step_ok(moe)
    except SystemExit as exc:
        # The overlapped dispatch did not come through its gate on this machine: say so and measure the
        # plainer form (push kernel + barrier before the owner's routing) instead of publishing nothing.
        if not (moe.peer is not None and moe.fuse_dispatch):
            raise
        from sparsebench_b200 import _C

        fallback_note = f"overlapped dispatch failed its gate ({exc}); measured with the separate push kernel instead"
        if rank == 0:
            print(fallback_note, file=sys.stderr)
        torch.cuda.synchronize()
        _C.device_status(device).zero_()
        moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=n_copies, exchange="peer",
                                fuse_return=moe.fuse_return, fuse_dispatch=False, micro_batches=moe.micro_batches,
                                micro_fractions=moe.micro_fractions)
        out, parity = first_step_ok(moe)

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
    # slot experts, routing (1 launch, 3 beyond 131072 slots), SDD, DSD, (pack | [push rows +] barrier), combine.
    route_launches = 1 if world * moe.capacity <= 131072 else 3
    fused_return = moe.peer is not None and moe.fuse_return
    fused_dispatch = moe.peer is not None and moe.fuse_dispatch
    if fused_dispatch:
        # sort, plan, push counts, barrier, owner layout, SDD with the pushes, DSD (+ return) [, push], barrier, combine
        launches_per_step = 9 if fused_return else 10
        dispatch_leg = "rows pushed by the owner's SDD kernel, tiles wait for the arrival flags of the 256-row segments their rows lie in"
        if moe.push_beside:
            launches_per_step += 1  # the push kernel on its own stream
            dispatch_leg = ("rows pushed by a kernel on a second stream beside the owner's SDD kernel, whose tiles wait "
                            "for the arrival flags of the 256-row segments their rows lie in")
    else:
        if moe.peer is not None:
            # sort, plan, push counts, push rows, barrier, owner layout, SDD, DSD (+ return) [, push rows], barrier, combine
            launches_per_step = 10 if fused_return else 11
        else:
            launches_per_step = 8 + route_launches
        dispatch_leg = "separate push kernel and a barrier before routing" if moe.peer is not None else "all-to-all collective"
    if moe.micro_batches > 1:
        launches_per_step = launches_per_step * moe.micro_batches + 1  # every part is a whole step, plus the concatenation
    with clock_sampler_cls(local) as clocks:
        ms_per_step = _timed_steps(step, flush, args.warmup, args.steps, world)
    value = world * cfg.useful_flops / (ms_per_step * 1e-3) / 1e12
    check_status(moe, device, world, "after the timed steps")

    # ---- e2e: public API with host buffers -----------------------------------------------------------
    dev_inputs = (dev.x, dev.expert_idx, dev.expert_weight)
    staging = PackedStaging([layer_in.x, layer_in.expert_idx, layer_in.expert_weight], device)
    staged_once = staging.device_buffer()
    staged_views = staging.views(staged_once)
    host_out = torch.empty_like(layer_in.x).pin_memory()
    def e2e_step() -> None:
        # `step` is the captured graph (or the eager call) over dev.x / dev.expert_idx / dev.expert_weight.
        staged_once.copy_(staging.host, non_blocking=True)
        for fixed, part in zip(dev_inputs, staged_views):
            fixed.copy_(part, non_blocking=True)
        result = step()
        host_out.copy_(graph_out if result is None else result, non_blocking=True)

    e2e_latency_ms = _timed_steps(e2e_step, flush, args.warmup, args.steps, world)  # one step alone, nothing overlapped
    e2e_ms = _pipelined_e2e_ms(step, lambda result: graph_out if result is None else result, dev_inputs, staging,
                               args.warmup, args.steps, world)
    check_status(moe, device, world, "after the end-to-end steps")
    h2d = sum(t.numel() * t.element_size() for t in (layer_in.x, layer_in.expert_idx, layer_in.expert_weight))
    d2h = host_out.numel() * host_out.element_size()
    host_link = host_link_gbs(device, world)

    # ---- per-stage times on this rank (eager, an event at every stage mark) ---------------------------
    # With micro-batches the stages of the parts interleave; the breakdown (and the roofline of the
    # dominant matmul) is then taken on the same step run whole.
    timed_moe = moe
    if moe.micro_batches > 1:
        moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=n_copies, exchange="peer",
                                fuse_return=timed_moe.fuse_return, fuse_dispatch=timed_moe.fuse_dispatch,
                                push_beside=timed_moe.push_beside)
    names: list[str] = []
    sums: dict[str, float] = {}
    iters = max(5, min(args.steps, 30))
    for it in range(iters + 2):
        if world > 1:
            dist.barrier()  # the ranks start the step together, as they do inside the timed graph replays
        flush_l2(flush)
        # About a millisecond of GPU time in front of the step: the eager launches below queue up behind it, so that
        # an event pair brackets device work and not the host's launch latency (a busy host inflated the stages).
        torch.cuda._sleep(2_000_000)
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
    # Every rank's matmul times and received rows: under skewed routing the step is as slow as its busiest owner.
    mine = torch.tensor([gemm_ms["sdd"], gemm_ms["dsd"], float(received), float(rows)], dtype=torch.float64, device=device)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(everyone, mine)
    else:
        everyone = [mine]
    table = torch.stack(everyone).cpu()
    per_rank_stats = {
        "sdd_ms": [round(v, 4) for v in table[:, 0].tolist()], "dsd_ms": [round(v, 4) for v in table[:, 1].tolist()],
        "rows_received": [int(v) for v in table[:, 2].tolist()], "rows_padded": [int(v) for v in table[:, 3].tolist()],
        "matmuls_ms_max_minus_mean": float((table[:, 0] + table[:, 1]).max() - (table[:, 0] + table[:, 1]).mean()),
    }
    largest_stage = max(stage_ms, key=stage_ms.get)
    roofline.update({
        "kernel": f"bsr_gemm_kernel<{dominant}> on rank 0", "peak_source": peak_kind, "launch_ms": gemm_ms[dominant],
        "algorithmic_bytes": gemm_bytes[dominant], "live_rows": rows, "rows_moved": rows_moved, "traffic": None,
        "traffic_note": "no DRAM counter capture of the multi-rank step exists (profilers never wrap a multi-rank command)",
        "stages_ms": stage_ms, "largest_stage_on_rank0": largest_stage, "per_rank": per_rank_stats,
        "all_to_all": {"useful_bytes_per_direction": payload,
                       "sent_bytes_per_direction": payload if moe.peer is not None else world * moe.capacity * cfg.d_model * 2,
                       "time_at_measured_nvlink_ms": payload / (NVLINK_GBS_PER_DIRECTION * 1e9) * 1e3},
    })

    # ---- context: the same step with NCCL all-to-all collectives as the exchange (eager, few steps) --------
    nccl_context = None
    if world > 1 and timed_moe.peer is not None and not getattr(args, "no_nccl_context", False):
        try:
            nccl_capacity = min(n_copies, int(math.ceil(factor * n_copies / world / 128.0)) * 128)
            nccl_moe = ExpertParallelMoE(dev.w1, dev.w2, cfg.num_experts, capacity=nccl_capacity, exchange="nccl")
            nccl_steps = min(args.steps, 10)
            nccl_ms = _timed_steps(lambda: nccl_moe(dev.x, dev.expert_idx, dev.expert_weight), flush, 3, nccl_steps, world)
            check_status(nccl_moe, device, world, "NCCL-exchange context steps")
            nccl_context = {"ms_per_step": nccl_ms, "value": world * cfg.useful_flops / (nccl_ms * 1e-3) / 1e12,
                            "steps": nccl_steps, "capacity_rows_per_pair": nccl_capacity,
                            "how": "same step, dispatch and return as fixed-capacity NCCL all-to-all collectives, eager launches"}
            del nccl_moe
        except SystemExit as exc:
            nccl_context = {"unavailable": str(exc)[:200]}

    line = {
        "metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(cfg, world),
        "method": {"parallelism": f"ep{world}", "experts_per_gpu": per_rank, "capacity_rows_per_pair": moe.capacity,
                   "exchange": exchange, "return_leg": "stored by the DSD epilogue" if fused_return else "separate kernel",
                   "dispatch_leg": dispatch_leg, "dispatch_fallback": fallback_note,
                   "micro_batches": timed_moe.micro_batches,
                   "micro_fractions": [round(f, 4) for f in timed_moe.micro_fractions],
                   "launch": launch, "l2": "256 MiB written and read back before every step (L2 cold and clean)",
                   "frac_of_bf16_peak": value / world / bf16_tflops},
        "parity": parity,
        "nccl_exchange": nccl_context,
        "clocks": clocks.summary(),
        "e2e": {"value": world * cfg.useful_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "steps pipelined over three streams (copy in, step, copy out), two sets of staging buffers; "
                       "every step's H2D and D2H copies are inside the timed region",
                "single_step_latency_ms": e2e_latency_ms, "host_link_all_ranks_copying": host_link,
                # What the host link allows: this rank's bytes per step over its share of the bidirectional rate.
                "host_link_floor_ms": (h2d + d2h) / (host_link["both_directions"]["slowest_rank_gbs"] * 1e9) * 1e3},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": roofline,
    }
    return line
