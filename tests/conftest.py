"""Shared fixtures. Tests marked ``gpu`` need a B200 and call the CUDA library through its C ABI; all others
run on the CPU (oracle against golden vectors, host logic, the allocator over a fake device, ABI checks)."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def oracle():
    from oracle_backend import OracleBackend
    return OracleBackend()


@pytest.fixture(scope="session")
def cuda():
    """The CUDA backend on device 0. No fallback: a missing library or device fails the test."""
    from homura_b200.host import CudaBackend
    backend = CudaBackend(0)
    yield backend
    backend.close()
