"""The library ships native sm_100a code for this GPU (reference: tests/test_smoke.py)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_kernel_runs_native_code_for_this_gpu() -> None:
    from sparsebench_b200 import _C

    out = _C.arch_probe(1000)  # not a multiple of the block size: the bounds check runs
    torch.cuda.synchronize()
    major, minor = torch.cuda.get_device_capability()
    assert out.shape == (1000,) and out.dtype == torch.int32
    assert torch.all(out == major * 100 + minor * 10).item()
    assert (major, minor) == (10, 0), "this library is built for sm_100a only"


def test_rejects_bad_size() -> None:
    from sparsebench_b200 import _C

    with pytest.raises(RuntimeError, match="must be positive"):
        _C.arch_probe(0)
