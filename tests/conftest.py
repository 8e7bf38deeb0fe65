import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(autouse=True, scope="session")
def _non_default_cuda_stream():
    """The library rejects the NULL (legacy default) stream, as the reference does
    (cpp/kernels/qwen35_attention.cu:430), so GPU tests make a real stream current."""
    try:
        import torch
    except ImportError:
        yield
        return
    if torch.cuda.is_available():
        torch.cuda.set_device(0)
        torch.cuda.set_stream(torch.cuda.Stream())
    yield
