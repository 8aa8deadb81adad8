import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "coda-gqa-l_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Make sure libcoda_b200.so exists before anything imports the package."""
    lib = os.path.join(ROOT, "coda-gqa-l_b200", "coda_gqa_l_b200", "libcoda_b200.so")
    if not os.path.exists(lib):
        sys.path.insert(0, os.path.join(ROOT, "coda-gqa-l_b200"))
        import build as _build
        _build.build()
    yield
