import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def pkg():
    """The engine package, with libgmlp.so built (nvcc cross-compiles without a GPU)."""
    entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def cuda_dev():
    import torch

    assert torch.cuda.is_available(), "GPU test collected without a GPU"
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _kernel_status_clean(request):
    """After every GPU test: no kernel may have given up a bounded wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        p = entry.load_package()
        import torch

        assert p._lib.status_read(torch.device("cuda:0")) == 0, "a kernel recorded a device-side timeout"
