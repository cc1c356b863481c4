"""The library-kernel context pipelines of bench_baselines.py compute the same layer as the oracle
(the reference checks its own baseline rows the same way, tests/test_baselines.py:26-41)."""

import pytest
import torch

import bench_baselines as B
from oracle import moe as M
from sparsebench_b200.workloads import LayerConfig, make_layer

CFG = LayerConfig("baseline_check", num_tokens=300, d_model=256, ffn_dim=256, num_experts=8, routing="zipf")


def expected_and_inputs(dtype: torch.dtype):
    layer = make_layer(CFG, seed=3, dtype=dtype)
    want = M.moe_reference(layer.x.float(), layer.expert_idx, layer.expert_weight.float(), layer.w1.float(),
                           layer.w2.float())
    return layer, want


@pytest.mark.parametrize("name", ["per_expert_loop", "padded_bmm"])
def test_pipeline_matches_oracle_on_cpu(name: str) -> None:
    layer, want = expected_and_inputs(torch.float32)
    got = B.PIPELINES[name](layer.x, layer.expert_idx, layer.expert_weight, layer.w1, layer.w2)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(B.PIPELINES))
def test_pipeline_matches_oracle_on_gpu(name: str) -> None:
    layer, want = expected_and_inputs(torch.bfloat16)
    dev = layer.to("cuda")
    try:
        got = B.PIPELINES[name](dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    except (RuntimeError, AttributeError) as exc:
        if name == "grouped_mm":
            pytest.skip(f"torch._grouped_mm is not usable here: {exc!r}")
        raise
    torch.testing.assert_close(got.float().cpu(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.gpu
def test_measure_reports_every_pipeline() -> None:
    from sparsebench_b200 import moe_forward
    from sparsebench_b200.timing import l2_flush_buffer

    dev = make_layer(CFG, seed=3).to("cuda")
    ours = moe_forward(dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    rows = B.measure(CFG, dev, l2_flush_buffer(), ours, iters=3)
    assert set(rows) == set(B.PIPELINES)
    for name, row in rows.items():
        assert "unavailable" in row or (row["ms"] > 0 and row["max_abs_diff_vs_ours"] < 0.1), (name, row)
