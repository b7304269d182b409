import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "understanding-gpu-architecture-implications-on-llm-serving-workloads_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("test marked gpu but no CUDA device is visible")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test: no kernel may have recorded an expired wait."""
    yield
    if request.node.get_closest_marker("gpu"):
        from b200k import _lib
        code, detail = _lib.device_status()
        assert code == 0, f"device status {code}, detail {detail:#x}"
