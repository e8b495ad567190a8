"""Bandwidth sweep of the fused chain (config 4): n = 2^20 ... 2^31 elements, f32 and bf16, kernel time per launch.

Method: per size, `iters` evaluations of the expression are queued behind enough L2-flush kernels that the host is
ahead of the GPU; every evaluation is bracketed by its own pair of events and followed by another L2 flush, so each
sample is one cold launch without host gaps. Inputs are a 2^20-element pattern tiled on the device (a row-broadcast
`contiguous`), which also gives a checksum: sum(z) must equal repeats x sum(z over the pattern).

    python -m aix_b200.sweep [max_log2n] [min_log2n]
"""
import json
import sys
import time

import numpy as np

from . import _capi as C
from .device import DeviceB200, to_storage
from .tensor import TensorValue, scalar_like

PATTERN = 1 << 20


def chain(a, b, c):
    one = lambda t: scalar_like(1.0, t)
    return (a * b + c) * (one(a) / (one(a) + (-a).exp())) - b.tanh() / (one(c) + (-c).exp())


def tiled(dev, pattern: TensorValue, repeats: int) -> TensorValue:
    if repeats == 1:
        return pattern.reshape((1, PATTERN))
    return pattern.reshape((1, PATTERN)).broadcastTo((repeats, PATTERN)).contiguous()


def measure(dev, log2n, dtype, iters=10):
    n = 1 << log2n
    repeats = n // PATTERN
    esize = C.DTYPE_SIZES[dtype]
    rng = np.random.default_rng(0)
    patterns = [TensorValue.from_numpy(rng.uniform(-1, 1, PATTERN).astype(np.float32), dev, dtype) for _ in range(3)]
    zp = chain(*[p.reshape((1, PATTERN)) for p in patterns])
    pattern_sum = float(zp.numpy().astype(np.float64).sum())
    a, b, c = (tiled(dev, p, repeats) for p in patterns)
    dev.synchronize()
    for _ in range(2):                       # warm-up: compile, populate the allocator cache
        z = chain(a, b, c)
        dev.synchronize()
    t0 = time.perf_counter()
    z = chain(a, b, c)
    host_s = time.perf_counter() - t0        # host cost of issuing one evaluation
    s = z.sum()
    checksum = float(s.item())
    del s
    events = [(dev.createEvent(), dev.createEvent()) for _ in range(iters)]
    blockers = int(1.5 * iters * (host_s + 60e-6) / 45e-6) + 4
    for _ in range(blockers):
        dev.flushL2()
    for e0, e1 in events:
        dev.recordEvent(e0)
        z = chain(a, b, c)
        dev.recordEvent(e1)
        dev.flushL2()
    ms = [dev.elapsedMs(e0, e1) for e0, e1 in events]
    for e0, e1 in events:
        dev.destroyEvent(e0); dev.destroyEvent(e1)
    best, med = float(np.min(ms)), float(np.median(ms))
    stats = dev.stats()
    del z, a, b, c
    dev.emptyCache()
    nbytes = 4 * n * esize
    want = pattern_sum * repeats
    return {"log2n": log2n, "dtype": C.DTYPE_NAMES[dtype], "bytes": nbytes, "ms_median": med, "ms_best": best,
            "GB/s_median": nbytes / (med * 1e-3) / 1e9, "GB/s_best": nbytes / (best * 1e-3) / 1e9,
            "host_us_per_evaluation": host_s * 1e6, "checksum": checksum, "checksum_expected": want,
            "checksum_rel_err": abs(checksum - want) / max(1.0, abs(want)), "kernels_total": stats["fused_kernels"]}


def run(dev, max_log2n=31, min_log2n=20, dtypes=(C.F32, C.BF16)):
    out = []
    for dtype in dtypes:
        for log2n in range(min_log2n, max_log2n + 1):
            if (4 + 13) * (1 << log2n) * C.DTYPE_SIZES[dtype] > 150 * (1 << 30):
                continue                     # would not fit next to the dead intermediates of one evaluation
            out.append(measure(dev, log2n, dtype, iters=10 if log2n < 28 else 5))
    return out


if __name__ == "__main__":
    hi = int(sys.argv[1]) if len(sys.argv) > 1 else 31
    lo = int(sys.argv[2]) if len(sys.argv) > 2 else 20
    device = DeviceB200(0)
    for rec in run(device, hi, lo):
        print(json.dumps(rec), flush=True)
    device.close()
