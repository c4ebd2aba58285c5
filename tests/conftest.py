import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a real B200 (run with -m gpu)")


def _gpu_usable() -> bool:
    try:
        import mind_b200.blas as blas
        return blas.device_count() > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def gpu():
    """The library on a usable B200; GPU tests fail (not skip) if it cannot load."""
    import mind_b200.blas as blas
    assert blas.device_count() > 0, "no sm_100 device visible to libmind_b200"
    return blas
