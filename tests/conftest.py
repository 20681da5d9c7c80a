import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the unmodified reference on seeded inputs (tests/golden/make_golden.py)."""
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "moe_golden.npz")))


@pytest.fixture(scope="session")
def port():
    """The plain-C restatement of the reference path (oracle/moe_oracle.c)."""
    import oracle
    oracle.build()
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    """The unmodified reference behind a C wrapper, where it was built."""
    import oracle
    if not oracle.have_ref():
        pytest.skip("oracle/_ref/libcsk_ref.so not built (needs the reference checkout)")
    return oracle.ref()


@pytest.fixture(scope="session")
def gpu_lib():
    """libcsk_moe.so on a B200; the GPU tests fail (not skip) if it cannot load."""
    from coalsack_b200 import _lib
    lib = _lib.load()
    assert lib.csk_moe_device_ok(0) == 1, "no usable sm_100 device"
    return lib
