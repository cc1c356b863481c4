"""Host-side behaviour that needs no GPU: argument checks of the operator mirror (the error text
the reference's TORCH_CHECKs give), the Python wrappers' ValueErrors, workload generators."""

import pytest
import torch

from sparsebench_b200 import _C, moe, spmm, workloads
from sparsebench_b200.topology import Topology


def test_package_exports_the_reference_surface() -> None:
    import sparsebench_b200 as sb

    for name in ("moe_forward", "route_device", "build_topology_cuda", "DeviceTopology", "sdd", "dsd", "Topology"):
        assert hasattr(sb, name)
    for name in ("arch_probe", "build_topology_cuda", "sdd_cuda", "dsd_cuda"):
        assert callable(getattr(_C, name))  # the four functions of the reference's extension module


@pytest.mark.parametrize(("make", "match"), [
    (lambda: torch.tensor([[0, 1]]), "CUDA"),  # reference: tests/test_routing.py:123-129
])
def test_routing_rejects_cpu_tensor(make, match: str) -> None:
    with pytest.raises(RuntimeError, match=match):
        _C.build_topology_cuda(make(), 8, 32, 16)


def _empty_topology(bs: int) -> Topology:
    z = torch.zeros(0, dtype=torch.int32)
    return Topology(bs, 4, 2, z, z, z, z, z, torch.zeros(1, dtype=torch.int32), z)


def test_sdd_wrapper_rejects_block_size_64() -> None:
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="block size 128"):
        spmm.sdd(x, torch.zeros(4, 128, 256, dtype=torch.bfloat16), _empty_topology(64))


def test_dsd_wrapper_rejects_block_shape_mismatch() -> None:
    with pytest.raises(ValueError, match="blocks must be"):
        spmm.dsd(torch.zeros(3, 64, 32, dtype=torch.bfloat16), torch.zeros(256, 128, dtype=torch.bfloat16),
                 _empty_topology(64))


def test_dsd_rejects_cpu_weights() -> None:
    with pytest.raises(RuntimeError, match="CUDA"):
        _C.dsd_cuda(torch.zeros(1, 128, 128, dtype=torch.bfloat16), torch.zeros(128, 128, dtype=torch.bfloat16),
                    torch.zeros(2, dtype=torch.int32), torch.zeros(1, dtype=torch.int32), 1)


def test_moe_forward_shape_errors() -> None:
    x = torch.zeros(5, 8, dtype=torch.bfloat16)
    w1, w2 = torch.zeros(4, 8, 256, dtype=torch.bfloat16), torch.zeros(4, 256, 8, dtype=torch.bfloat16)
    idx, gate = torch.zeros(5, 2, dtype=torch.int64), torch.zeros(5, 2, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="w2 must be"):
        moe.moe_forward(x, idx, gate, w1, w2.transpose(1, 2))
    with pytest.raises(ValueError, match="x must be"):
        moe.moe_forward(x, idx, gate[:, :1], w1, w2)


def test_arch_probe_rejects_bad_size_before_touching_a_device() -> None:
    with pytest.raises(RuntimeError, match="must be positive"):
        _C.arch_probe(0)


def test_workloads_are_seeded_and_distinct() -> None:
    for name in workloads.CASE_NAMES + ["permuted_zipf"]:
        a, b = workloads.routing_case(name, 64, 16, seed=3), workloads.routing_case(name, 64, 16, seed=3)
        assert torch.equal(a, b) and a.shape == (64, 2) and a.dtype == torch.int64
        assert torch.all(a[:, 0] != a[:, 1]) and int(a.min()) >= 0 and int(a.max()) < 16
    z = workloads.routing_case("zipf", 4096, 64)
    pz = workloads.routing_case("permuted_zipf", 4096, 64)
    # Zipf: expert 0 is the busiest; the permuted variant moves the head somewhere else but keeps the shape.
    cz, cpz = torch.bincount(z.reshape(-1), minlength=64), torch.bincount(pz.reshape(-1), minlength=64)
    assert int(cz.argmax()) == 0 and torch.equal(cz.sort().values[-4:] > 400, torch.ones(4, dtype=torch.bool))
    assert abs(int(cz.max()) - int(cpz.max())) < 400


def test_layer_config_flops_and_shapes() -> None:
    cfg = workloads.CONFIGS["fine_grained"]
    assert cfg.useful_flops == 4 * 4096 * 2 * 1024 * 4096  # 137.4 GFLOP
    small = workloads.LayerConfig("t", 16, 64, 256, 4, "random")
    layer = workloads.make_layer(small, seed=1)
    assert layer.x.shape == (16, 64) and layer.w1.shape == (4, 64, 256) and layer.w2.shape == (4, 256, 64)
    assert layer.x.dtype == torch.bfloat16 and layer.expert_idx.dtype == torch.int64
    assert torch.allclose(layer.expert_weight.float().sum(-1), torch.ones(16), atol=2e-2)
    again = workloads.make_layer(small, seed=1)
    assert torch.equal(layer.x, again.x) and torch.equal(layer.w2, again.w2)
    other_tokens = workloads.make_layer(small, seed=1, token_seed=5)
    assert torch.equal(layer.w1, other_tokens.w1) and not torch.equal(layer.x, other_tokens.x)


def test_expert_parallel_argument_errors() -> None:
    # Without a process group the layer is a single rank: the peer exchange options have nothing to act on.
    from sparsebench_b200.ep import ExpertParallelMoE

    w1, w2 = torch.zeros(4, 64, 256, dtype=torch.bfloat16), torch.zeros(4, 256, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="micro_batches"):
        ExpertParallelMoE(w1, w2, 4, micro_batches=2)
    with pytest.raises(ValueError, match="micro_batches"):
        ExpertParallelMoE(w1, w2, 4, micro_batches=0)
    with pytest.raises(ValueError, match="exchange"):
        ExpertParallelMoE(w1, w2, 4, exchange="mpi")
    with pytest.raises(ValueError, match="do not split"):
        ExpertParallelMoE(w1, w2, 8)
    with pytest.raises(ValueError, match="w2_local"):
        ExpertParallelMoE(w1, w2.transpose(1, 2), 4)
