import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def synth(pkg):
    return pkg.synth


@pytest.fixture(scope="session")
def port():
    from oracle.oracle_py import Oracle
    return Oracle("port")


@pytest.fixture(scope="session")
def ref():
    from oracle.oracle_py import Oracle, ref_available
    if not ref_available():
        pytest.skip("oracle/_ref/libfm_ref.so not built (no reference checkout on this machine)")
    return Oracle("reference")
