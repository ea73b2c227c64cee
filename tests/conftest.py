import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device; run with -m gpu")


@pytest.fixture(scope="session")
def ora():
    """The CPU oracle (test infrastructure)."""
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def ctx():
    """One device context for the whole GPU session."""
    import juliavision_b200 as jv
    c = jv.Ctx(0)
    yield c
    c.close()


def relerr(got, ref):
    """max|got-ref| / max|ref|, the reference tests' error measure (test_flash.jl:142)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))


def poison(ctx, arr):
    """Fill an output with 0xff bytes (NaN in fp16/fp32) so unwritten elements show up."""
    ctx.fill_bytes(arr, 0xFF)
