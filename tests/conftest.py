import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box with -m gpu)")


@pytest.fixture(scope="session")
def port():
    """The CPU restatement (oracle/liboracle.so), built on demand with g++."""
    from oracle import oracle
    if not oracle.available("port"):
        oracle.build()
    return oracle.load("port")


@pytest.fixture(scope="session")
def reference():
    """The reference project's own CPU templates (oracle/_ref), if they were built where a checkout exists."""
    from oracle import oracle
    if not oracle.available("reference"):
        pytest.skip("oracle/_ref/libsimnets_ref.so not built (needs a checkout of the reference project)")
    return oracle.load("reference")


@pytest.fixture(scope="session")
def cuda_lib():
    """The CUDA library; on a GPU box a missing build is an error, never a skip."""
    from simnets_tf_b200 import _lib
    return _lib.lib()
