import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_oracle():
    import oracle
    oracle.build()


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    # a fresh checkout has no libcombskv.so (built artefacts are not tracked): compile it once, where nvcc exists
    from combsengine_b200 import _build
    if not os.path.exists(_build.LIB):
        _build.build()
