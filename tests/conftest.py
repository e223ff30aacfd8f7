import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Files whose GPU tests run with guard zones around every CUDA tensor the test creates through torch.zeros / empty / full
# / *_like (llmq_b200/utils/guards.py): a kernel that writes past its output fails the test instead of silently changing a
# neighbouring tensor.  (compute-sanitizer is not available for these runs; this is the bounds check that always runs.)
_GUARDED = ("test_kernels_gpu.py", "test_mx_gpu.py", "test_fused_emulated_gpu.py", "test_zz_no_alloc.py")


@pytest.fixture(autouse=True)
def _guard_device_buffers(request):
    import torch

    if "gpu" not in request.keywords or not torch.cuda.is_available() or request.node.fspath.basename not in _GUARDED:
        yield
        return
    from llmq_b200.utils.guards import guard_torch_allocations

    with guard_torch_allocations("cuda"):
        yield
        torch.cuda.synchronize()
