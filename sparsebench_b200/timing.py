"""GPU timing shared by the benchmark and the tests, so every number is measured the same way
(the reference's sparsebench/timing.py): CUDA events on the launching stream, L2 flushed before
every timed call so each one starts cold."""

from __future__ import annotations

import statistics
from collections.abc import Callable

import torch

L2_FLUSH_BYTES = 256 * 1024 * 1024  # B200's L2 is 126 MB; the reference's 128 MB buffer would not clear it


def l2_flush_buffer(device: torch.device | str = "cuda") -> torch.Tensor:
    return torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)


def flush_l2(buffer: torch.Tensor) -> None:
    """Empties L2 of everything the timed code could hit: writes the whole buffer (twice the size of L2),
    then reads it back once. The write alone would leave L2 full of DIRTY lines, and the first ~20 us
    of whatever is timed next would pay for writing 126 MB of them back to HBM; after the read pass L2
    holds clean lines of the buffer only. Enqueued on the current stream; no sync."""
    buffer.zero_()
    torch.sum(buffer.view(torch.int64))


def time_each_ms(fn: Callable[[], object], flush: torch.Tensor | None, warmup: int = 3, iters: int = 20,
                 leave_l2_dirty: bool = False) -> list[float]:
    """GPU time of every one of `iters` calls of fn(), in ms. Events are recorded on torch's
    current stream, which is the stream the kernels are launched on. leave_l2_dirty: flush by the
    write pass alone (the reference's way), so that fn() also pays for the write-back of an L2 full of
    dirty lines."""
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(iters):
        if flush is not None:
            if leave_l2_dirty:
                flush.zero_()
            else:
                flush_l2(flush)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        samples.append(start.elapsed_time(end))
    return samples


def time_ms(fn: Callable[[], object], flush: torch.Tensor | None, warmup: int = 3, iters: int = 20) -> float:
    """Median GPU time of fn() in ms."""
    return statistics.median(time_each_ms(fn, flush, warmup, iters))


def marginal_stage_times_ms(stages: list[tuple[str, Callable[[dict], None]]], flush: torch.Tensor | None,
                            warmup: int = 3, iters: int = 20) -> dict[str, float]:
    """GPU time in ms of every stage of a pipeline IN ITS PLACE in the pipeline: the graph of the first
    j stages is timed for j = 0..n (CUDA events around each replay, L2 flushed before it), and stage j
    gets the difference between prefix j and prefix j-1. Every prefix ends with the same one-element
    kernel, so that each graph ends the same way (a small kernel waiting for its predecessor to
    finish) whatever its last stage is; prefix 0 is that kernel alone. The one-off latency of launching
    a graph and the cost of the closing kernel are the same in every prefix and cancel, each stage runs
    after its real predecessor with the cache state that predecessor leaves, and nothing is inserted
    between the stages. Each stage is a callable that reads and writes a shared dict."""
    closing = torch.zeros(1, device="cuda")
    means: list[float] = []
    for j in range(len(stages) + 1):
        def run(j: int = j) -> dict:
            state: dict = {}
            for _, stage in stages[:j]:
                stage(state)
            closing.add_(1.0)
            return state

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = run()
        means.append(statistics.mean(time_each_ms(graph.replay, flush, warmup, iters)))
        del graph, keep
    return {name: means[j + 1] - means[j] for j, (name, _) in enumerate(stages)}
