import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _check_tensor_core_errors():
    """After every GPU test, fail if a tensor-core kernel reported that one of its bounded waits ran out."""
    yield
    try:
        import torch

        if torch.cuda.is_available():
            from hivemind_b200.ops.gemm import check_kernel_errors

            check_kernel_errors()
    except ImportError:
        pass
