import os
import pathlib
import subprocess
import sys

import pytest

REPO = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (oracle/liboracle.so), built on demand with its Makefile."""
    import oracle_lib

    return oracle_lib.load()


@pytest.fixture(scope="session")
def reference_kernels():
    """The reference's own CUDA kernels compiled from its sources (oracle/_ref), or a skip."""
    import oracle_lib

    library = oracle_lib.load_reference()
    if library is None:
        pytest.skip("oracle/_ref/libmmh3_ref.so has not been built")
    return library
