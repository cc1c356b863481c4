"""Expert-parallel parity on the benchmark's own shape, on as many GPUs as this machine has.

Launches tests/ep_multi_gpu.py under torchrun for N = 2, 4 and 8 ranks (skipped where the machine has
fewer GPUs): E=128 experts, D=F=2048, T=4096 tokens per rank, permuted-Zipf routing, capacity T*k, in the
form the benchmark uses at that N and with the dispatch overlapped inside the owner's SDD kernel. Every rank checks its own
4096 output rows against the fp32 oracle on its tokens with all 128 experts (rtol = atol = 2e-2), eagerly
and through a replayed CUDA graph with new tokens and routing, and the owner's layout against the
single-process layout of the concatenated batch.
"""

from __future__ import annotations

import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(world: int, mode: str, size: str, timeout_s: int = 900) -> str:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "ep_multi_gpu.py"),
           mode, size]
    proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout_s)
    text = proc.stdout + proc.stderr
    assert proc.returncode == 0, "\n".join(text.splitlines()[-40:])
    return text


@pytest.mark.parametrize("form", ["bench", "bench_overlapped"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_benchmark_shape_matches_oracle_on_every_rank(world: int, form: str) -> None:
    # "bench": the form the benchmark runs at this rank count; "bench_overlapped": the dispatch inside the owner's
    # SDD kernel, whole step, whatever the benchmark's default is.
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this machine has {torch.cuda.device_count()}")
    text = _launch(world, form, "full")
    for rank in range(world):
        assert f"rank {rank}/{world}: expert-parallel parity ok" in text, text[-3000:]


# "peer": dispatch overlapped, the push kernel on a second stream beside SDD; "peer_warps": pushed by SDD's own warps;
# "peer_nodispatch": separate push kernel and barrier; "peer_unfused": two-kernel return; "peer_mb2": two micro-batches;
# "peer_split": two micro-batches of a quarter and three quarters of the tokens.
@pytest.mark.parametrize("mode", ["nccl", "peer", "peer_warps", "peer_unfused", "peer_nodispatch", "peer_mb2", "peer_split"])
def test_other_exchange_modes_small_shape(mode: str) -> None:
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    text = _launch(2, mode, "small")
    assert "rank 1/2: expert-parallel parity ok" in text, text[-3000:]
