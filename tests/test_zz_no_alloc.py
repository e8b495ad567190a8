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
        # and against the exact value of what the device holds: float64 for floats, the wrapping integer sum for i32
        held = t.numpy()
        exact = held.astype(np.int64).sum().astype(np.int32) if dtype == I32 else held.astype(np.float64).sum()
        assert_close(first.numpy(), np.asarray(exact, dtype=first.numpy().dtype), dtype, f"against the exact sum n={n}", scale=scale)
        assert np.array_equal(first.numpy(), second.numpy()), "same grid, same fold order: the two calls agree to the bit"


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


def test_static_scratch_sum_waits_for_a_collective_in_flight_on_its_operand(b200):
    """An overlapped all-reduce may still be running on the operand: the sum is ordered after it, as every other entry
    point is (one rank is enough to see the ordering - the collective and its scaling pass run on a side stream)."""
    from aix_b200 import DeviceB200
    b200.commInit(0, 1, DeviceB200.commUniqueId())
    try:
        host = np.full(1 << 22, 2.0, dtype=np.float32)
        t = TensorValue.from_numpy(host, b200)
        out = TensorValue.empty((), b200, F32)
        b200.synchronize()
        b200.allReduceAsync(t.storage.data, t.size, F32, 0.25)       # sum over one rank, then x 0.25 on the side stream
        b200.sumStaticScratch(t.deviceParams(), out.deviceParams())
        assert float(out.numpy()) == 0.5 * (1 << 22)
    finally:
        b200.commDestroy()
