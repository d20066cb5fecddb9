import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def golden():
    d = os.path.join(ROOT, "tests", "golden")

    def load(family):
        z = np.load(os.path.join(d, family + "_kat.npz"))
        return z["table"], z["data"]
    return load


def ulp_diff(a, b):
    """Distance in units in the last place between two float32 arrays (the reference's
    SNN_ALMOST_EQUAL, test/helpers/float_comparison.h:264-293)."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def rel_err(got, ref):
    """The relative error the parity tolerances are stated in, taken two ways and the larger returned:
    the max-norm  max |got - ref| / max |ref|,  and the element-wise  max_i |got_i - ref_i| /
    (|ref_i| + rms(ref)).  The second keeps one large output from hiding errors on the small ones:
    rel_err <= tol means |got_i - ref_i| <= tol * |ref_i| + tol * rms(ref) for every element."""
    got = np.asarray(got, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    diff = np.abs(got - ref)
    scale = max(float(np.max(np.abs(ref))), 1e-30)
    rms = max(float(np.sqrt(np.mean(ref * ref))), 1e-30)
    return max(float(np.max(diff)) / scale, float(np.max(diff / (np.abs(ref) + rms))))
