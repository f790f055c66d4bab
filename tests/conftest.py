import os
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(REPO, "sparse-dropout_b200")
for p in (PKG, REPO):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(REPO, "tests", "golden", "reference_golden.npz"))


@pytest.fixture(scope="session")
def built_lib():
    """libsparsedrop.so, built on demand (nvcc cross-compiles for sm_100a without a GPU)."""
    from flash_dropout import _lib
    if not os.path.exists(_lib.LIB_PATH):
        import subprocess
        subprocess.check_call(["sh", os.path.join(PKG, "csrc", "build.sh")], stdout=subprocess.DEVNULL,
                              stderr=subprocess.DEVNULL)
    return _lib.lib()
