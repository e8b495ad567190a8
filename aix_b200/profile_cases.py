"""Small, fixed workloads for profiler captures: each case runs ONE kernel class a few times on inputs that are larger
than the 126 MB L2 but hold well under a few GB on the device.

    python -m aix_b200.profile_cases <case> [repeats]

cases: chain_f32 chain_bf16 chain_sum_f32 chain_sum_bf16 config1_bf16 sum_f32 sum_bf16 rowsum_bf16 rowmax_bf16 colsum_f32 gemm_bf16_nt gemm_bf16_nn gemm_bf16_tn gemm_f32
       gemm_bf16_k1024 gemm_f32_4096 gemm_f32_4096_nt gemm_f32_4096_tn gemm_f32_k1024 adam_f32 mlp_f32
Prints the device time per repeat measured with events on the device's stream.
"""
import sys

import numpy as np

from . import _capi as C
from .device import DeviceB200
from .tensor import TensorValue, scalar_like


def _rand(dev, shape, dtype, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return TensorValue.from_numpy((rng.uniform(-1, 1, shape) * scale).astype(np.float32), dev, dtype)


def chain(a, b, c):
    one = lambda t: scalar_like(1.0, t)
    return (a * b + c) * (one(a) / (one(a) + (-a).exp())) - b.tanh() / (one(c) + (-c).exp())


def build(dev, case):
    if case.startswith("chain_"):
        dt = C.F32 if case.endswith("f32") else C.BF16
        a, b, c = (_rand(dev, (1 << 16, 1024), dt, s) for s in range(3))
        if case.startswith("chain_sum_"):
            def both():                                   # the sum is recorded behind the chain: one kernel
                z = chain(a, b, c)
                return z, z.sum()
            return both
        return lambda: chain(a, b, c)
    if case == "config1_bf16":
        # configuration 1 as the API issues it: y = relu(x*g + bias), y.sum(1), y.max(1), y.mean() - one row-form kernel
        x = _rand(dev, (8192, 8192), C.BF16, 0)
        g, b = _rand(dev, (8192,), C.BF16, 1), _rand(dev, (8192,), C.BF16, 2, 0.1)

        def whole():
            v = x * g + b
            y = (v + (v * v).sqrt()) * 0.5
            return y, y.sum(1), y.max(1), y.mean()
        return whole
    if case in ("sum_f32", "sum_bf16"):
        x = _rand(dev, (1 << 17, 1024), C.F32 if case.endswith("f32") else C.BF16, 0)
        return lambda: x.sum()
    if case in ("rowsum_bf16", "rowmax_bf16"):
        x = _rand(dev, (16384, 8192), C.BF16, 0)
        return (lambda: x.sum(1)) if case.startswith("rowsum") else (lambda: x.max(1))
    if case == "colsum_f32":
        x = _rand(dev, (16384, 4096), C.F32, 0)
        return lambda: x.sum(0)
    if case in ("gemm_f32_4096_nt", "gemm_f32_4096_tn"):
        # the backward forms of the 4096^3 f32 product: G . B^T (all K-major) and A^T . G (both operands MN-major)
        a, b = _rand(dev, (4096, 4096), C.F32, 0, 0.05), _rand(dev, (4096, 4096), C.F32, 1, 0.05)
        return (lambda: a.matmul(b.transpose(0, 1))) if case.endswith("_nt") else (lambda: a.transpose(0, 1).matmul(b))
    if case in ("gemm_f16_4096", "gemm_bf16_k12288"):
        # probes: the f16 form of the 16-bit kernel, and a contraction three times as long (the depth of the three f32 passes)
        dt = C.F16 if case.startswith("gemm_f16") else C.BF16
        k = 12288 if case.endswith("k12288") else 4096
        a, b = _rand(dev, (4096, k), dt, 0, 0.05), _rand(dev, (4096, k), dt, 1, 0.05)
        return lambda: a.matmul(b.transpose(0, 1))
    if case in ("gemm_bf16_k1024", "gemm_f32_k1024", "gemm_f32_4096"):
        # the MLP's shapes: batch 4096, a 1024-wide or 4096-wide contraction
        dt = C.BF16 if "bf16" in case else C.F32
        k = 1024 if case.endswith("k1024") else 4096
        a, b = _rand(dev, (4096, k), dt, 0, 0.05), _rand(dev, (k, 4096), dt, 1, 0.05)
        return lambda: a.matmul(b)
    if case == "mlp_f32":
        from .mlp import MlpTrainer
        trainer = MlpTrainer(dev)
        return trainer.step
    if case.startswith("gemm_"):
        dt = C.F32 if case == "gemm_f32" else C.BF16
        n = 2048 if dt == C.F32 else 4096
        a, b = _rand(dev, (n, n), dt, 0, 0.05), _rand(dev, (n, n), dt, 1, 0.05)
        if case.endswith("_nt"): return lambda: a.matmul(b.transpose(0, 1))
        if case.endswith("_tn"): return lambda: a.transpose(0, 1).matmul(b)
        return lambda: a.matmul(b)
    if case == "adam_f32":
        p, g, m, v = (_rand(dev, (1 << 16, 1024), C.F32, s) for s in range(4))

        def step():
            m2 = 0.9 * m + 0.1 * g
            v2 = 0.999 * v * v + 0.001 * g * g
            return p - (0.001 * (m2 / 0.1) / ((v2 / 0.001).sqrt() + 1e-8)), m2, v2
        return step
    raise SystemExit(f"unknown case {case}")


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "chain_f32"
    repeats = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    dev = DeviceB200(0)
    fn = build(dev, case)
    dev.synchronize()
    marker = dev.createEvent()
    for _ in range(3):                   # warm-up: kernels compiled and loaded, allocator cache populated
        out = fn()
        dev.recordEvent(marker)          # emits the recorded work per call, as the timed loop does (else the calls merge into other kernels)
    dev.synchronize()
    e0, e1 = dev.createEvent(), dev.createEvent()
    dev.flushL2()
    dev.recordEvent(e0)
    for _ in range(repeats):
        out = fn()
        dev.recordEvent(e1)
    ms = dev.elapsedMs(e0, e1) / repeats
    stats = dev.stats()
    print(f"{case}: {ms:.4f} ms per repeat over {repeats} repeats (one event pair around all repeats: the device queue stays "
          f"full); launches so far {stats['total_kernel_launches']}")
    del out
    dev.close()


if __name__ == "__main__":
    main()
