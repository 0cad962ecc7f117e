import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # The CPU checker and the CUDA library are compiled, git-ignored artefacts: (re)build them when their sources
    # are newer.  Both builds are incremental and need no GPU (nvcc cross-compiles).
    from oracle import oracle as O
    O.build()
    from denograd_b200 import build as B
    try:
        B.build()
    except RuntimeError:
        if not os.path.exists(B.LIB):
            raise


@pytest.fixture(scope="session")
def dev():
    from denograd_b200 import Device
    return Device["CUDA"]
