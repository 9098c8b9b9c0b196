import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import cpu_oracle
    return cpu_oracle.Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle import cpu_oracle
    if not cpu_oracle.reference_available():
        try:
            cpu_oracle.build()
        except Exception:
            pass
    if not cpu_oracle.reference_available():
        pytest.skip("compiled reference (oracle/_ref/libtbn_ref.so) not available")
    return cpu_oracle.Reference()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    d = os.path.join(ROOT, "tests", "golden")
    return {n[:-4]: np.load(os.path.join(d, n)) for n in os.listdir(d) if n.endswith(".npz")}
