import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def b200():
    """The device under test, through the C ABI. Fails (does not skip) when the library or the GPU is missing."""
    from aix_b200 import DeviceB200
    dev = DeviceB200(0)
    yield dev
    dev.synchronize()
    dev.close()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU device (oracle/_ref, built from the reference sources)."""
    from oracle.ref_device import DeviceRefCPU, available
    if not available():
        pytest.skip("oracle/_ref/libaixref.so not built (reference sources absent)")
    return DeviceRefCPU()


@pytest.fixture(scope="session")
def dry():
    """A B200 device that records, plans and compiles but never touches a GPU."""
    from aix_b200 import DeviceB200
    dev = DeviceB200(0, dry_run=1, disk_cache=0)
    yield dev
    dev.close()


def tolerance(dtype):
    """Relative tolerance per element type: integers exact, f32 1e-5, f16/bf16 1e-2, f64 1e-12."""
    from aix_b200 import BF16, F16, F32, F64
    return {F64: 1e-12, F32: 1e-5, F16: 1e-2, BF16: 1e-2}.get(dtype, 0.0)


def assert_close(actual, expected, dtype, what="", scale=None):
    actual = np.asarray(actual)
    expected = np.asarray(expected)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} vs {expected.shape}"
    tol = tolerance(dtype)
    if tol == 0.0:
        assert np.array_equal(actual, expected), f"{what}: integer results differ at {np.argwhere(actual != expected)[:5].tolist()}"
        return
    a = actual.astype(np.float64)
    e = expected.astype(np.float64)
    both_nan = np.isnan(a) & np.isnan(e)
    same_inf = np.isinf(a) & np.isinf(e) & (np.sign(a) == np.sign(e))
    ref_scale = np.maximum(1.0, np.abs(e)) if scale is None else scale
    with np.errstate(invalid="ignore"):
        bad = ~(both_nan | same_inf | (np.abs(a - e) <= tol * ref_scale))
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} differ beyond {tol}; first at {np.argwhere(bad)[:3].tolist()} "
                           f"got {a[bad][:3]} want {e[bad][:3]}")
