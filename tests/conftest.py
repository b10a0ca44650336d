import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with `-m gpu` on the GPU box")


@pytest.fixture(scope="session", autouse=True)
def built_libraries():
    """The CUDA library and the oracle are built before any test loads them. On the GPU box the
    prebuilt files travel with the tree and nothing is rebuilt."""
    import oracle_lib
    from modelspec_b200 import _build

    if not os.path.exists(_build.LIB):
        _build.build_library()
    if not os.path.exists(os.path.join(oracle_lib.ORACLE_DIR, "liboracle.so")):
        oracle_lib.build()


@pytest.fixture(scope="session")
def device():
    import modelspec_b200 as M

    d = M.Device(0)
    yield d
    d.close()
