"""Failure handling, with every failure made on the host (nothing here faults, traps or hangs a GPU).

Reference behaviour being matched: allocation retries after the caches have been emptied and then throws
std::runtime_error (aixDeviceMetal.cpp:1433-1475); a kernel that cannot be compiled is reported (the reference prints
and drops the op, aixDeviceMetalKernelGen.cpp:737-743 - here the call fails with the compiler's message and the device
stays usable). The GPU part makes a bounded device-side wait run out through the library's own self-test kernel: the
kernel returns normally, the next synchronize reports a timeout, and the device works afterwards."""
import numpy as np
import pytest

from aix_b200 import F32, DeviceB200, TensorValue

MB = 1 << 20


def test_injected_out_of_memory_is_retried_after_trimming_then_reported():
    dev = DeviceB200(0, dry_run=1, disk_cache=0, inject_alloc_limit_bytes=64 * MB)
    a = TensorValue.empty((12 * MB,), dev, F32)          # 48 MiB live
    b = TensorValue.empty((2 * MB,), dev, F32)           # + 8 MiB
    del b                                                # parked in the allocator's cache
    c = TensorValue.empty((3 * MB,), dev, F32)           # 12 MiB: does not fit beside the cached block -> trim, retry, succeed
    stats = dev.stats()
    assert stats["bytes_cached"] == 0 and stats["bytes_in_use"] >= 60 * MB
    with pytest.raises(RuntimeError, match="failed after emptying the cache"):
        TensorValue.empty((4 * MB,), dev, F32)           # 16 MiB more: over the injected limit even with an empty cache
    del c
    d = TensorValue.empty((3 * MB,), dev, F32)           # the device is usable afterwards
    d.fill(1.0)
    dev.synchronize()
    del a, d
    dev.close()


def test_dead_buffers_behind_recorded_ops_are_released_by_a_flush_before_giving_up():
    dev = DeviceB200(0, dry_run=1, disk_cache=0, inject_alloc_limit_bytes=80 * MB)
    x = TensorValue.full(1.0, (4 * MB,), dev)            # blocks are 18 MiB each (16 MiB + headroom, 2 MiB pages)
    y = x + 1.0                                          # + the filled scalar operand (dead at once, but parked behind the recorded ops) + y
    before = dev.stats()
    assert before["bytes_in_use"] == 54 * MB and before["flushes"] == 0
    z = y * 2.0                                          # scalar operand: 72 MiB; z: 90 MiB > limit -> emit the recorded ops, which
    after = dev.stats()                                  # returns the first scalar operand's block, and retry
    assert after["flushes"] == 1 and after["bytes_in_use"] == 72 * MB and after["bytes_reserved"] == 72 * MB
    dev.synchronize()
    del x, y, z
    dev.close()


def test_injected_compiler_failure_is_reported_and_the_device_stays_usable():
    dev = DeviceB200(0, dry_run=1, disk_cache=0, inject_nvrtc_failures=1)
    x = TensorValue.full(2.0, (1000,), dev)
    with pytest.raises(RuntimeError, match="NVRTC failed to compile a fused kernel"):
        dev.synchronize()
    assert "extern \"C\" __global__" in dev.lastKernelSource()      # the source that failed is kept for inspection
    misses = dev.stats()["kernel_cache_misses"]
    y = TensorValue.full(2.0, (1000,), dev)              # the same kernel again: compiled now, not served from a poisoned cache
    dev.synchronize()
    assert dev.stats()["nvrtc_compiles"] == 1 and dev.stats()["kernel_cache_misses"] == misses + 1
    dev.close()


@pytest.mark.gpu
def test_a_bounded_device_wait_that_runs_out_is_reported_once_and_the_device_recovers(b200):
    x = TensorValue.from_numpy(np.arange(1000, dtype=np.float32), b200)
    b200.synchronize()
    b200.selfTestBoundedWait(1_000_000)                  # 1 ms limit on a barrier nobody arrives at
    y = x + 1.0                                          # work queued behind the self-test still runs
    with pytest.raises(TimeoutError, match="bounded device-side wait ran out"):
        b200.synchronize()
    b200.synchronize()                                   # reported once
    assert np.array_equal(y.numpy(), np.arange(1000, dtype=np.float32) + 1.0)
    m = TensorValue.from_numpy(np.ones((256, 256), np.float32), b200).matmul(TensorValue.from_numpy(np.ones((256, 256), np.float32), b200))
    assert np.all(m.numpy() == 256.0)                    # the tensor-core path (which shares the error word) is unaffected


# ---- communicator failures, injected on the host (no NCCL, no GPU): aixb200_comm_inject_backend -----------------------
@pytest.fixture()
def injected():
    from aix_b200 import _capi as C
    lib = C.load()

    def counters():
        import ctypes
        a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        lib.aixb200_comm_injected_counters(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return {"inits": a.value, "polls": b.value, "aborts": c.value}
    yield lib, counters
    lib.aixb200_comm_inject_backend(0, 0)
    import os
    os.environ.pop("AIXB200_COMM_INIT_TIMEOUT_MS", None)


def test_a_rank_that_never_joins_costs_a_timeout_and_one_abort(injected, monkeypatch):
    import time
    lib, counters = injected
    monkeypatch.setenv("AIXB200_COMM_INIT_TIMEOUT_MS", "150")
    assert lib.aixb200_comm_inject_backend(1, 0) == 0                   # initialisation stays "in progress" for ever
    dev = DeviceB200(0, dry_run=1, disk_cache=0)
    t0 = time.time()
    with pytest.raises(TimeoutError, match="did not complete within 150 ms"):
        dev.commInit(0, 2, b"\0" * 128)
    assert 0.1 <= time.time() - t0 < 5.0
    seen = counters()
    assert seen["inits"] == 1 and seen["aborts"] == 1 and seen["polls"] > 10
    x = TensorValue.full(1.0, (100,), dev)                              # the device itself is unaffected
    dev.synchronize()
    with pytest.raises(Exception, match="comm_init"):
        dev.allReduce(x.storage.data, x.size, F32, 1.0)                 # no communicator came into being; nothing is aborted twice
    assert counters()["aborts"] == 1
    dev.commDestroy()
    dev.close()


def test_an_asynchronous_error_aborts_the_communicator_once(injected, monkeypatch):
    lib, counters = injected
    monkeypatch.setenv("AIXB200_COMM_INIT_TIMEOUT_MS", "2000")
    assert lib.aixb200_comm_inject_backend(2, 3) == 0                   # healthy for three status queries, then a remote error
    dev = DeviceB200(0, dry_run=1, disk_cache=0)
    dev.commInit(0, 2, b"\0" * 128)                                     # query 1: ready
    x = TensorValue.full(1.0, (100,), dev)
    dev.allReduce(x.storage.data, x.size, F32, 1.0)                     # query 2 (comm_wait) and 3 (all_reduce): still healthy
    with pytest.raises(RuntimeError, match="asynchronous NCCL error.*aborted"):
        dev.synchronize()                                               # query 4: the error surfaces at the next call
    assert counters()["aborts"] == 1
    with pytest.raises(RuntimeError, match="aborted after an earlier failure"):
        dev.allReduce(x.storage.data, x.size, F32, 1.0)
    dev.commDestroy()                                                   # no second abort, no destroy of an aborted communicator
    assert counters()["aborts"] == 1
    dev.close()


def test_blocking_initialisation_stays_the_default(injected):
    lib, counters = injected
    assert lib.aixb200_comm_inject_backend(2, 1000) == 0
    dev = DeviceB200(0, dry_run=1, disk_cache=0)
    dev.commInit(0, 1, b"\0" * 128)
    assert counters() == {"inits": 1, "polls": 0, "aborts": 0}          # plain ncclCommInitRank: nothing to poll
    dev.commDestroy()
    dev.close()
