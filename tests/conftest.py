"""pytest configuration: the `gpu` marker and the import path.

`-m "not gpu"` runs the oracle against the golden vectors, the host logic and the C-ABI symbol
checks on any machine; `-m gpu` runs the parity tests proper on a B200 through the C ABI.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (NVIDIA B200, sm_100a)")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA GPU")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_status_stays_clean(request: pytest.FixtureRequest):
    """After every GPU test: no matmul kernel may have given up on one of its bounded waits."""
    yield
    if "gpu" not in request.keywords:
        return
    import torch

    from sparsebench_b200 import _C

    for index, status in list(_C._dev_status.items()):
        value = int(status.item())
        if value != 0:
            status.zero_()
            pytest.fail(f"device status word on cuda:{index} is {value}: a bounded device-side wait expired")
