"""bench.py's reference arm and argument handling run without a GPU: the JSON line has the keys the
contract names."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_the_contract_keys() -> None:
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "cpu_small",
                           "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["config"]["workload"] == "cpu_small" and line["n_gpus"] == 1
    # "reference": the reference's own reference.py from the copy under baseline/_ref; "port": the oracle.
    have_copy = (ROOT / "baseline" / "_ref" / "sparsebench_ref" / "reference.py").exists()
    assert line["cpu_baseline"]["kind"] == ("reference" if have_copy else "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["steps"] == 2 and set(line["config"]) == {"workload", "tokens", "d_model", "ffn_dim", "experts", "top_k",
                                                          "routing", "block_size"}
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["gpu_launches"] == 0


def test_non_zero_ranks_of_the_reference_arm_do_no_work() -> None:
    env = {"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1", "PATH": "/usr/bin:/bin"}
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                          capture_output=True, text=True, timeout=120, env={**__import__("os").environ, **env})
    assert proc.returncode == 0 and proc.stdout.strip() == ""


def test_expert_parallel_form_follows_the_flags_and_the_measured_table() -> None:
    # Which form of the peer-exchange step the benchmark runs: --ep-dispatch wins, the older flag means "separate",
    # otherwise the per-rank-count table; every listed rank count has a micro-batch default of at least one.
    import types

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench_ep

    def wanted(world: int, **flags) -> bool:
        return bench_ep.overlapped_dispatch_wanted(types.SimpleNamespace(**flags), world)

    for world, (overlapped, micro_batches) in bench_ep.DEFAULT_EP_FORM.items():
        assert wanted(world) is overlapped and wanted(world, ep_dispatch="auto") is overlapped
        assert micro_batches >= 1 and bench_ep.DEFAULT_MICRO_BATCHES[world] == micro_batches
    assert wanted(3) is False, "rank counts without a measurement run the plainest form"
    for world in (2, 4, 8):
        assert wanted(world, ep_dispatch="overlapped") and wanted(world, ep_dispatch="beside")
        assert not wanted(world, ep_dispatch="separate")
        assert not wanted(world, ep_dispatch="overlapped", ep_unfused_dispatch=True)
