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


def time_each_ms(fn: Callable[[], object], flush: torch.Tensor | None, warmup: int = 3, iters: int = 20) -> list[float]:
    """GPU time of every one of `iters` calls of fn(), in ms. Events are recorded on torch's
    current stream, which is the stream the kernels are launched on."""
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
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


def captured(fn: Callable[[], object]) -> tuple[torch.cuda.CUDAGraph, object]:
    """fn() captured into a CUDA graph (after one eager call on a side stream, so that one-time
    set-up stays outside the capture). Returns (graph, fn's result): keep the result alive as long as
    the graph is replayed. Replaying puts the kernels on the GPU with no host work in between, so
    events around graph.replay() time the kernels and not the Python and driver calls that launch them."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        result = fn()
    return graph, result
