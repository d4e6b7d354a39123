import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_gpu() -> bool:
    try:
        from novann_b200.device import device_count
        return device_count() > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def gpu():
    """Device 0, or a hard failure: GPU tests never skip into a CPU path."""
    if not _has_gpu():
        pytest.fail("no CUDA device / libnvq.so missing: GPU tests cannot run")
    return 0


@pytest.fixture(scope="session")
def oracle_c():
    from oracle import oracle_c as oc
    return oc.load()
