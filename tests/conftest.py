import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


@pytest.fixture(scope="session")
def native_library():
    """The built C-ABI library (built on demand with nvcc; no GPU needed to build)."""
    from anemoi_b200.build import build

    build()
    from anemoi_b200 import native

    return native.library()
