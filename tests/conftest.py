import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu on the GPU box")


def _has_gpu() -> bool:
    try:
        import magnetron_b200 as mb
        return mb.device_count() > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def gpu():
    """Device ordinal 0 of the C-ABI library; GPU tests fail (not skip) when the library is missing."""
    import magnetron_b200 as mb
    mb.lib()  # raises if the CUDA library was not built: never fall back
    if mb.device_count() < 1:
        pytest.fail("no sm_100 device visible: GPU tests must run on a B200")
    mb.check(mb.lib().magb200_device_init(0))
    return 0
