import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA GPU (B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def oracle_c():
    """The plain-C oracle (oracle/librz_oracle.so), built on demand with gcc."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "librz_oracle.so")
    src = os.path.join(ROOT, "oracle", "rz_oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")])
    return ctypes.CDLL(path)


@pytest.fixture(scope="session")
def rzlib():
    """The product library; built on demand when nvcc is present (never replaced by a fallback)."""
    from rzlinear_b200 import _lib, build
    if build.needs_build():
        build.build()
    return _lib
