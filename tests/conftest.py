import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # Rebuild the C-ABI library when a source is newer than it (no-op otherwise), so the tests
    # never exercise a stale binary.
    import shutil
    if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
        import setup_runtime
        setup_runtime.build()


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
