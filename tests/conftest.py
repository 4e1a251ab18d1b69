import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Make sure the oracle and the library exist (both are prebuilt in-tree on a GPU box)."""
    if not os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so")):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
    if not os.path.exists(os.path.join(ROOT, "sptmm_b200", "libsptmm.so")):
        subprocess.run([sys.executable, os.path.join(ROOT, "sptmm_b200", "build.py")], check=True)


def has_gpu() -> bool:
    try:
        import sptmm_b200
        return sptmm_b200.device_count() > 0
    except Exception:
        return False
