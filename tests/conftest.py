import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def port_lib():
    from oracle import build_oracle
    from oracle import np_oracle as O

    return O.PortLib(build_oracle.build_port())


@pytest.fixture(scope="session")
def ref_lib():
    """The reference's compiled I2_S kernel, when it has been built (needs a checkout at
    build time; the built file is reused on machines without one)."""
    from oracle import build_oracle
    from oracle import np_oracle as O

    path = build_oracle.build_ref()
    if not path:
        pytest.skip("compiled reference not available")
    return O.RefLib(path)
