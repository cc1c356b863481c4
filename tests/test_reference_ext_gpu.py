"""This library's kernels against the REFERENCE's own CUDA kernels on the same GPU.

oracle/build_ref_ext.py compiles the reference's unmodified CUDA sources for sm_100 into
oracle/_ref/sparsebench_ref_C.so (git-ignored; skipped here when it has not been built or does not
load). It is a second oracle beside the CPU one: routing must agree with the reference's
build_topology_cuda in every output buffer bit for bit, worst-case tails and error word included; SDD,
DSD and the layer must agree within the tolerance of two bf16 pipelines (1.6e-2, the reference's own).
"""

import pytest
import torch

from oracle.build_ref_ext import load_ref_ext
from sparsebench_b200.workloads import CONFIGS, LayerConfig, make_layer
from tests.cases import CASE_NAMES, routing_case

pytestmark = pytest.mark.gpu

NAMES = ("tokens_per_expert", "padded_offsets", "row_token", "copy_row", "row_block_expert", "row_offsets",
         "col_indices", "error")


@pytest.fixture(scope="module")
def ref():
    ext, why = load_ref_ext()
    if ext is None:
        pytest.skip(why)
    return ext


@pytest.mark.parametrize("case", CASE_NAMES)
@pytest.mark.parametrize(("num_tokens", "num_experts", "block_size"), [(13, 8, 16), (1000, 64, 128), (4096, 64, 128),
                                                                       (3000, 256, 4), (100_000, 1024, 128)])
def test_routing_buffers_equal_the_reference_kernels(ref, case: str, num_tokens: int, num_experts: int,
                                                      block_size: int) -> None:
    from sparsebench_b200 import _C

    idx = routing_case(case, num_tokens, num_experts).cuda()
    ffn_dim = 2 * block_size
    want = ref.build_topology_cuda(idx, num_experts, ffn_dim, block_size)
    got = _C.build_topology_cuda(idx, num_experts, ffn_dim, block_size)
    for name, a, b in zip(NAMES, got, want):
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert torch.equal(a, b), f"{name} differs from the reference's kernel"


def test_routing_bad_ids_equal_the_reference_kernels(ref) -> None:
    from sparsebench_b200 import _C

    idx = routing_case("random", 500, 8, seed=3).cuda()
    idx[7, 0], idx[123, 1], idx[499, 0] = -1, 8, 1 << 40
    for dtype in (torch.int64, torch.int32):
        ids = idx.clamp(-1, 1 << 20).to(dtype) if dtype == torch.int32 else idx
        want = ref.build_topology_cuda(ids, 8, 256, 128)
        got = _C.build_topology_cuda(ids, 8, 256, 128)
        for name, a, b in zip(NAMES, got, want):
            assert torch.equal(a, b), f"{name} differs from the reference's kernel ({dtype})"
        assert int(got[-1].item()) == 1


@pytest.mark.parametrize("name", ["cpu_small", "fine_grained_zipf"])
def test_matmuls_and_layer_agree_with_the_reference_kernels(ref, name: str) -> None:
    from bench_baselines import reference_gpu_forward
    from sparsebench_b200 import _C, moe_forward

    cfg = CONFIGS[name]
    dev = make_layer(cfg, seed=0).to("cuda")
    topo = _C.build_topology_cuda(dev.expert_idx, cfg.num_experts, cfg.ffn_dim, 128)
    _, offsets, row_token, _, row_block_expert, row_offsets, col_indices, _ = topo
    live_blocks = int(offsets[-1].item()) // 128 * (cfg.ffn_dim // 128)
    h_ref = ref.sdd_cuda(dev.x, dev.w1, row_token, row_block_expert, row_offsets, col_indices.numel(), True)
    h = _C.sdd_cuda(dev.x, dev.w1, row_token, row_block_expert, row_offsets, col_indices.numel(), True)
    torch.testing.assert_close(h[:live_blocks].float(), h_ref[:live_blocks].float(), rtol=1.6e-2, atol=1.6e-2)
    w2_cat = dev.w2.view(cfg.num_experts * cfg.ffn_dim, cfg.d_model)
    live_rows = int(offsets[-1].item())
    y_ref = ref.dsd_cuda(h_ref, w2_cat, row_offsets, col_indices, 5)
    y = _C.dsd_cuda(h_ref, w2_cat, row_offsets, col_indices, 5)
    torch.testing.assert_close(y[:live_rows].float(), y_ref[:live_rows].float(), rtol=1.6e-2, atol=1.6e-2)
    args = (dev.x, dev.expert_idx, dev.expert_weight, dev.w1, dev.w2)
    torch.testing.assert_close(moe_forward(*args).float(), reference_gpu_forward(ref)(*args).float(), rtol=2e-2, atol=2e-2)
