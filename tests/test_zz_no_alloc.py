"""Allocation-free sum (aixb200_sum_static_scratch): for callers that cannot allocate at call time - a fixed memory
budget, a region where cudaMalloc is not allowed, a device owned by another allocator. Its partial sums live in a
static device array of the library instead of heap scratch. Checked through the C ABI against the regular
aixb200_sum on two calls in a row (the array keeps the previous call's contents), plus its refusals.
Collected last on purpose: a failure here must not hide the rest of the suite under -x."""
import numpy as np
import pytest

from aix_b200 import BF16, DTYPE_NAMES, F32, F64, I32, DeviceTensorParams, TensorValue
from conftest import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [F32, BF16, F64, I32], ids=lambda d: DTYPE_NAMES[d])
def test_static_scratch_sum_matches_regular_sum_twice_in_a_row(b200, dtype):
    rng = np.random.default_rng(41 + dtype)
    for n in (1, 1000, (1 << 20) + 3):
        x = rng.integers(-50, 50, n) if dtype == I32 else rng.normal(0, 1, n)
        t = TensorValue.from_numpy(x, b200, dtype)
        regular = t.sum()
        first = TensorValue.empty((), b200, dtype)
        second = TensorValue.empty((), b200, dtype)
        b200.synchronize()
        mallocs = b200.stats()["cuda_mallocs"]
        b200.sumStaticScratch(t.deviceParams(), first.deviceParams())
        b200.sumStaticScratch(t.deviceParams(), second.deviceParams())      # reuses the array left by the first call
        assert b200.stats()["cuda_mallocs"] == mallocs
        want = regular.numpy()
        scale = max(1.0, float(np.abs(np.asarray(x, dtype=np.float64)).sum()))
        assert_close(first.numpy(), want, dtype, f"first call n={n}", scale=scale)
        assert_close(second.numpy(), want, dtype, f"second call n={n}", scale=scale)


def test_static_scratch_sum_refusals(b200):
    t = TensorValue.from_numpy(np.ones(16, dtype=np.float32), b200)
    out = TensorValue.empty((), b200, F32)
    b200.synchronize()
    host = np.ones(16, dtype=np.float32)
    with pytest.raises(ValueError, match="device memory"):
        b200.sumStaticScratch(DeviceTensorParams(host.ctypes.data, F32, 0, (16,), 16, (1,)), out.deviceParams())
    too_big = (1 << 30) + 1
    with pytest.raises(ValueError, match="at most"):
        b200.sumStaticScratch(DeviceTensorParams(t.storage.data, F32, 0, (too_big,), too_big, (1,)), out.deviceParams())
    u = t + 1.0                                  # recorded, not flushed
    with pytest.raises(ValueError, match="pending"):
        b200.sumStaticScratch(t.deviceParams(), out.deviceParams())
    b200.synchronize()
    b200.sumStaticScratch(u.deviceParams(), out.deviceParams())
    assert out.numpy() == 32.0
