import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _strict_kernels_on_gpu(request, monkeypatch):
    """GPU tests must hit the CUDA kernels: a silent PyTorch fallback is an error there."""
    if request.node.get_closest_marker("gpu") is not None:
        monkeypatch.setenv("KMOE_STRICT", "1")
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from kolmogorov_moe_architecture_b200.ops import cuda_ops
            cuda_ops.check_status()
