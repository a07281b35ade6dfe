import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


# the tests switch kernels through environment variables between calls; the library
# otherwise reads them once per process
os.environ.setdefault("KS_B200_ENV_RELOAD", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device; run with -m gpu")


@pytest.fixture(scope="session")
def ks():
    """The product package. Importing it loads libkernel_set.so (built on demand)."""
    lib = os.path.join(ROOT, "kernel_set_b200", "lib", "libkernel_set.so")
    if not os.path.exists(lib):
        from kernel_set_b200.build import build
        build()
    import kernel_set_b200
    return kernel_set_b200


@pytest.fixture(scope="session")
def cuda(ks):
    """cuda:0 with the CUDA library path armed; a GPU test on a machine without
    a usable device fails loudly instead of being skipped."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device is visible"
    assert torch.cuda.get_device_capability(0)[0] == 10, "these tests need an sm_100 device"
    return torch.device("cuda:0")
