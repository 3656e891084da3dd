"""Shared fixtures.  `-m "not gpu"` runs everywhere; `-m gpu` needs a B200."""
import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


@pytest.fixture(scope="session")
def hb():
    """The ctypes binding of libhb.so (built on demand; nvcc needs no GPU)."""
    entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def kats():
    with open(ROOT / "tests" / "golden" / "reference_kats.json") as f:
        return json.load(f)


@pytest.fixture(scope="session")
def cuda(hb):
    import torch

    if hb.device_count() < 1 or not torch.cuda.is_available():
        pytest.fail("this test is marked gpu but no CUDA device is visible; libhb has no CPU path")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
