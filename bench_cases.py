#!/usr/bin/env python
"""Measurement cases beside bench.py: the secondary kernel-class measurements its JSON line carries (`extras`, `mlp_train`,
`config1_sharded`), the small fixed workloads the profiler captures under profiles/ were taken on, and the bandwidth sweep
of the fused chain. Nothing of the device library imports this file.

    python bench_cases.py <case> [repeats]         one kernel class a few times on inputs larger than L2 but well under a few GB;
                                                   prints the device time per repeat (events on the device's stream). Cases:
        chain_f32 chain_bf16 chain_sum_f32 chain_sum_bf16 config1_bf16 sum_f32 sum_bf16 rowsum_bf16 rowmax_bf16 colsum_f32
        gemm_bf16_nt gemm_bf16_nn gemm_bf16_tn gemm_f32 gemm_bf16_k1024 gemm_f32_4096 gemm_f32_4096_nt gemm_f32_4096_tn
        gemm_f32_k1024 gemm_f16_4096 gemm_bf16_k12288 adam_f32 mlp_f32
    python bench_cases.py sweep [max_log2n] [min_log2n]    chain bandwidth for n = 2^min ... 2^max, f32 and bf16
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from aix_b200 import _capi as C                                      # noqa: E402
from aix_b200.device import DeviceB200, to_storage                  # noqa: E402
from aix_b200.tensor import TensorValue, scalar_like                # noqa: E402

def chain(a, b, c):
    """z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c)) as the front end issues it (16 device calls)."""
    one = lambda t: scalar_like(1.0, t)
    return (a * b + c) * (one(a) / (one(a) + (-a).exp())) - b.tanh() / (one(c) + (-c).exp())


# ---- measurements carried by bench.py's JSON line --------------------------------------------------------------------
def _time(dev, fn, iters=10, warmup=3, flush_l2=True):
    """Device time of one call of fn. The calls are issued from Python, whose per-call cost (tens of microseconds) can
    exceed a kernel's duration; to keep the interval between the two events free of host time, enough L2-flush kernels
    (about 45 us each) are queued first that the host finishes issuing all `iters` calls while the GPU is still busy
    with them. The host cost per call is measured during the warm-up. The working sets used here (>= 128 MiB per
    call) do not fit the L2 together with the next call's."""
    import time
    marker = dev.createEvent()
    host_s = 0.0
    for _ in range(warmup):
        t0 = time.perf_counter()
        fn()
        dev.recordEvent(marker)
        host_s = max(host_s, time.perf_counter() - t0)
    dev.synchronize()
    e0, e1 = dev.createEvent(), dev.createEvent()
    head = min(400, 3 + int(1.5 * iters * host_s / 45e-6))
    for _ in range(head if flush_l2 or head > 3 else 1):
        dev.flushL2()
    dev.recordEvent(e0)
    for _ in range(iters):
        fn()
        dev.recordEvent(marker)         # flushes recorded elementwise work: one launch set per call, as in a real step
    dev.recordEvent(e1)
    ms = dev.elapsedMs(e0, e1) / iters
    dev.destroyEvent(marker)
    dev.destroyEvent(e0)
    dev.destroyEvent(e1)
    return float(ms), float(host_s * 1e3)


def relu(v):
    return (v + (v * v).sqrt()) * 0.5


def measure_reductions(dev, hbm_peak, rows=8192, cols=8192):
    rng = np.random.default_rng(0)
    x = TensorValue.from_numpy(rng.normal(0, 1, (rows, cols)).astype(np.float32), dev, C.BF16)
    g = TensorValue.from_numpy(rng.uniform(0.5, 1.5, cols).astype(np.float32), dev, C.BF16)
    b = TensorValue.from_numpy(rng.normal(0, 0.1, cols).astype(np.float32), dev, C.BF16)
    dev.synchronize()
    n = rows * cols
    out = {}
    holder = {}

    y = relu(x * g + b)
    dev.synchronize()

    def whole():
        # configuration 1 exactly as the API issues it: the device folds the row sums, the row maxima and the global sum
        # into the kernel that produces y (x read once, y written once); only the scalar division of the mean remains
        yy = relu(x * g + b)
        holder["all"] = (yy, yy.sum(1), yy.max(1), yy.mean())

    api_bytes = 5 * n * 2 + 2 * cols * 2            # y written + read by each of the three reductions, x read: 640 MiB
    moved_bytes = 2 * n * 2 + 2 * cols * 2          # what the fused form has to move: x in, y out
    med, host_ms = _time(dev, whole)
    out["config 1 whole (y, row sum, row max, mean) bf16"] = {
        "ms": med, "GB/s_of_API_bytes": api_bytes / (med * 1e-3) / 1e9, "GB/s_of_bytes_moved": moved_bytes / (med * 1e-3) / 1e9,
        "frac_of_measured_hbm_on_bytes_moved": moved_bytes / (med * 1e-3) / 1e9 / hbm_peak, "api_bytes": api_bytes,
        "bytes_moved": moved_bytes, "host_ms_per_call": host_ms}
    cases = {
        "relu(x*g+bias) bf16 [fused, y written]": (lambda: holder.__setitem__("y", relu(x * g + b)), 2 * n * 2 + 2 * cols * 2),
        "row sum bf16 (reduceTo)": (lambda: holder.__setitem__("s", y.sum(1)), n * 2),
        "row max bf16 (maxTo)": (lambda: holder.__setitem__("m", y.max(1)), n * 2),
        "global sum bf16": (lambda: holder.__setitem__("t", y.sum()), n * 2),
    }
    for name, (fn, nbytes) in cases.items():
        med, host_ms = _time(dev, fn)
        out[name] = {"ms": med, "GB/s": nbytes / (med * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (med * 1e-3) / 1e9 / hbm_peak,
                     "bytes": nbytes, "host_ms_per_call": host_ms}
    return out


def measure_matmul(dev, tensor_peak, size=4096):
    rng = np.random.default_rng(0)
    out = {}
    for name, dtype in (("bf16", C.BF16), ("f32", C.F32)):
        a = TensorValue.from_numpy(rng.normal(0, 0.02, (size, size)).astype(np.float32), dev, dtype)
        b = TensorValue.from_numpy(rng.normal(0, 0.02, (size, size)).astype(np.float32), dev, dtype)
        dev.synchronize()
        holder = {}
        forms = {"A.B": lambda: a.matmul(b), "G.B^T": lambda: a.matmul(b.transpose(0, 1)), "A^T.G": lambda: a.transpose(0, 1).matmul(b)}
        for form, fn in forms.items():
            med, _host = _time(dev, lambda: holder.__setitem__("c", fn()), iters=5, warmup=2, flush_l2=False)
            tf = 2.0 * size ** 3 / (med * 1e-3) / 1e12
            out[f"{name} {form} {size}^3"] = {"ms": med, "TFLOP/s": tf, "frac_of_measured_bf16_peak": tf / tensor_peak}
    return out


def measure_mlp(dev, tensor_peak, steps=10, warmup=3, rank=0, world_size=1, batch=4096, barrier=None, reduce_max=None, overlap=True,
                sharded=False, deferred=False, early=False):
    """MLP training configuration: device time of `steps` steps (forward, backward, gradient all-reduce when
    world_size > 1, Adam), loss not read inside the timed region."""
    from aix_b200.mlp import MlpTrainer
    trainer = MlpTrainer(dev, batch=batch, rank=rank, world_size=world_size, overlap=overlap, sharded=sharded, deferred=deferred, early=early)
    for _ in range(warmup):
        loss = trainer.step()
    first = float(loss.value.item())
    e0, e1 = dev.createEvent(), dev.createEvent()
    if barrier: barrier()
    dev.synchronize()
    s0 = dev.stats()
    dev.recordEvent(e0)
    import time
    issue_start = time.perf_counter()
    for _ in range(steps):
        loss = trainer.step()
    dev.recordEvent(e1)
    host_ms = (time.perf_counter() - issue_start) * 1e3 / steps        # time the host needs to issue a step (no wait for the device in it)
    ms = dev.elapsedMs(e0, e1)
    if barrier: barrier()
    if reduce_max: ms = reduce_max(ms)
    s1 = dev.stats()
    last = float(loss.value.item())
    per_step = ms / steps
    tf = trainer.flops_per_step / (per_step * 1e-3) / 1e12
    return {"config": "4 Linear 1024-4096-4096-4096-1024, tanh, f32, batch %d per GPU, MSE, Adam(1e-3)" % batch,
            "ms_per_step": per_step, "host_issue_ms_per_step": host_ms, "steps_per_s": 1e3 / per_step, "samples_per_s": world_size * batch * 1e3 / per_step,
            "gemm_TFLOP/s_per_gpu": tf, "frac_of_measured_bf16_peak": tf / tensor_peak, "world_size": world_size,
            "kernel_launches_per_step": (s1["total_kernel_launches"] - s0["total_kernel_launches"]) / steps,
            "fused_kernels_per_step": (s1["fused_kernels"] - s0["fused_kernels"]) / steps,
            "device_calls_per_step": (s1["ops_recorded"] - s0["ops_recorded"]) / steps,
            "prepared_operand_builds_per_step": (s1["prepared_operand_builds"] - s0["prepared_operand_builds"]) / steps,
            "prepared_operand_hits_per_step": (s1["prepared_operand_hits"] - s0["prepared_operand_hits"]) / steps,
            "gradient_exchange": "none" if world_size == 1 else (
                ("reduce-scatter per gradient started inside backward, each rank updates 1/N of every parameter, all-gather" +
                 ("; later layers' updates deferred into the next forward pass" if deferred else "") +
                 ("; first layers' updates and all-gathers moved into backward" if deferred and early else "")) if sharded
                else ("all-reduce per parameter, started inside backward" if overlap else "all-reduce per parameter after backward")),
            "loss_after_warmup": first, "loss_at_end": last}


def measure_cold_ops(dev, hbm_peak, n=10_000_000):
    """The remaining aix::Device virtuals at the size the reference's own device benchmarks use (10 M f32 elements,
    Targets/AIXBenchmarks/Device.cpp; transpose at its 5000 x 5000): device time per call and the rate of the bytes each
    call has to move. They are off the hot path; the figures say how far."""
    rng = np.random.default_rng(0)
    out, holder = {}, {}
    x = TensorValue.from_numpy(rng.normal(0, 1, n).astype(np.float32), dev)
    sq = TensorValue.from_numpy(rng.normal(0, 1, (5000, 5000)).astype(np.float32), dev)
    rows = TensorValue.from_numpy(rng.normal(0, 1, (10000, 1000)).astype(np.float32), dev)
    idx = TensorValue.from_numpy(rng.integers(0, 10000, 10000), dev, C.I32)
    few = TensorValue.from_numpy(rng.normal(0, 1, (64, 1000)).astype(np.float32), dev)
    idx_few = TensorValue.from_numpy(rng.integers(0, 64, 10000), dev, C.I32)
    r32 = TensorValue.empty((), dev, C.I32)
    onehot = TensorValue.empty((n,), dev, C.I32)
    sq_t = TensorValue.empty((5000, 5000), dev)
    sel = TensorValue.empty((10000, 1000), dev)
    tri = TensorValue.empty((5000, 5000), dev)
    dev.synchronize()
    cases = {
        "argmax 10M f32": (lambda: dev.argmax(x.deviceParams(), r32.deviceParams()), 4 * n),
        "argmaxIndices 10M f32": (lambda: dev.argmaxIndices(x.deviceParams(), onehot.deviceParams()), 8 * n),
        "max 10M f32": (lambda: holder.__setitem__("m", x.max()), 4 * n),
        "transpose 5000x5000 f32 (materialised)": (lambda: dev.transpose(sq.deviceParams(), sq_t.deviceParams(), 0, 1), 8 * 25_000_000),
        "contiguous of a transposed 5000x5000 view": (lambda: holder.__setitem__("c", sq.transpose(0, 1).contiguous()), 8 * 25_000_000),
        "tril 5000x5000 f32": (lambda: dev.tril(sq.deviceParams(), tri.deviceParams(), 0), 8 * 25_000_000),
        "indexSelect 10000 rows of 1000 f32": (lambda: dev.indexSelect(rows.deviceParams(), sel.deviceParams(), idx.deviceParams(), 0), 8 * n),
        "indexAdd 10000 rows of 1000 f32 into 10000 rows (atomics, whole slices as runs)": (lambda: dev.indexAdd(sel.deviceParams(), rows.deviceParams(), idx.deviceParams(), 0), 12 * n),
        "indexAdd 10000 rows of 1000 f32 into 64 rows (the same, ~156 additions per element)": (lambda: dev.indexAdd(sel.deviceParams(), few.deviceParams(), idx_few.deviceParams(), 0), 4 * n),
        "sliceSet 5000x2500 into every other column": (lambda: dev.sliceSet(TensorValue(sq.storage, (5000, 2500), (2500, 1), 0, C.F32, dev).deviceParams(),
                                                                              tri.deviceParams(), 1, 0, 5000, 2), 8 * 12_500_000),
    }
    for name, (fn, nbytes) in cases.items():
        ms, _host = _time(dev, fn, iters=5, warmup=2)
        out[name] = {"ms": ms, "GB/s": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm_peak}
    return out


def measure_extras(dev, hbm_peak, tensor_peak):
    return {"reductions_8192x8192_bf16": measure_reductions(dev, hbm_peak), "matmul": measure_matmul(dev, tensor_peak),
            "cold_ops_10M": measure_cold_ops(dev, hbm_peak)}


def measure_config1_sharded(dev, hbm_peak, rank, world_size, rows=8192, cols=8192, barrier=None, reduce_max=None):
    """Configuration 1 with the rows split across the ranks (weak scaling: every rank holds rows x cols): y, the row sums
    and the row maxima are local - one generated kernel - and the global mean takes one scalar all-reduce over NCCL.
    Returns per-GPU and aggregate rates; the mean is checked against the ranks' local means."""
    from aix_b200.frontend import global_mean
    rng = np.random.default_rng(rank)
    x = TensorValue.from_numpy(rng.normal(0, 1, (rows, cols)).astype(np.float32), dev, C.BF16)
    g = TensorValue.from_numpy(np.random.default_rng(1000).uniform(0.5, 1.5, cols).astype(np.float32), dev, C.BF16)
    b = TensorValue.from_numpy(np.random.default_rng(1001).normal(0, 0.1, cols).astype(np.float32), dev, C.BF16)
    dev.synchronize()
    holder = {}

    def whole():
        y = relu(x * g + b)
        holder["all"] = (y, y.sum(1), y.max(1), global_mean(y, world_size))

    for _ in range(3):
        whole()
    dev.synchronize()
    if barrier: barrier()
    iters = 10
    e0, e1 = dev.createEvent(), dev.createEvent()
    for _ in range(8):
        dev.flushL2()                      # keeps the device busy while the host queues the timed calls
    dev.recordEvent(e0)
    for _ in range(iters):
        whole()
    dev.recordEvent(e1)
    ms = dev.elapsedMs(e0, e1) / iters
    if reduce_max: ms = reduce_max(ms)
    y, _, _, mean = holder["all"]
    local_mean = float(y.numpy().astype(np.float64).mean())
    moved = 2 * rows * cols * 2 + 2 * cols * 2
    api = 5 * rows * cols * 2 + 2 * cols * 2
    return {"rows_per_gpu": rows, "cols": cols, "ms": ms, "GB/s_per_gpu_of_bytes_moved": moved / (ms * 1e-3) / 1e9,
            "GB/s_aggregate_of_bytes_moved": world_size * moved / (ms * 1e-3) / 1e9,
            "GB/s_aggregate_of_API_bytes": world_size * api / (ms * 1e-3) / 1e9,
            "frac_of_measured_hbm_per_gpu": moved / (ms * 1e-3) / 1e9 / hbm_peak,
            "global_mean": float(mean.numpy()), "local_mean_of_this_rank": local_mean, "exchange": "one scalar all-reduce per evaluation"}


# ---- fixed workloads for profiler captures -----------------------------------------------------------------------------
def _rand(dev, shape, dtype, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return TensorValue.from_numpy((rng.uniform(-1, 1, shape) * scale).astype(np.float32), dev, dtype)


def build_case(dev, case):
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
    if case in ("linear_values_f32_k1024", "linear_values_f32_k4096"):
        # matmul(x, W) + b on tensor values: the product is a temporary, so the add runs in its epilogue and only the sum is written
        k = 1024 if case.endswith("k1024") else 4096
        x, w, b = _rand(dev, (4096, k), C.F32, 0), _rand(dev, (k, 4096), C.F32, 1, 0.05), _rand(dev, (1, 4096), C.F32, 2, 0.1)
        return lambda: x.matmul(w) + b
    if case in ("linear_tanh_values_f32_k1024", "linear_tanh_values_f32_k4096"):
        # the same layer on tensor values, product and sum dropped as temporaries: the add runs in the product's epilogue, and
        # with AIXB200_GEMM_EPILOGUE=2 the tanh too
        k = 1024 if case.endswith("k1024") else 4096
        x, w, b = _rand(dev, (4096, k), C.F32, 0), _rand(dev, (k, 4096), C.F32, 1, 0.05), _rand(dev, (1, 4096), C.F32, 2, 0.1)
        return lambda: (x.matmul(w) + b).tanh()
    if case in ("linear_tanh_f32_k1024", "linear_tanh_f32_k4096"):
        # one hidden layer of the MLP as the front end issues it: matmul(x, W) + b, then tanh, all three results kept
        # (autograd holds them); with AIXB200_GEMM_EPILOGUE=0 the add and the tanh run as a generated kernel of their own
        k = 1024 if case.endswith("k1024") else 4096
        x, w, b = _rand(dev, (4096, k), C.F32, 0), _rand(dev, (k, 4096), C.F32, 1, 0.05), _rand(dev, (1, 4096), C.F32, 2, 0.1)

        def layer():
            mm = x.matmul(w)
            s = mm + b
            return mm, s, s.tanh()
        return layer
    if case == "mlp_f32":
        from aix_b200.mlp import MlpTrainer
        trainer = MlpTrainer(dev)
        return trainer.step
    if case.startswith("gemm_"):
        dt = C.F32 if case == "gemm_f32" else C.BF16
        n = 2048 if dt == C.F32 else 4096
        a, b = _rand(dev, (n, n), dt, 0, 0.05), _rand(dev, (n, n), dt, 1, 0.05)
        if case.endswith("_nt"): return lambda: a.matmul(b.transpose(0, 1))
        if case.endswith("_tn"): return lambda: a.transpose(0, 1).matmul(b)
        return lambda: a.matmul(b)
    if case in ("transpose_f32_5000", "tril_f32_5000"):
        # two of the data-movement virtuals at the size of the reference's device benchmarks
        sq = _rand(dev, (5000, 5000), C.F32, 0)
        out = TensorValue.empty((5000, 5000), dev)
        if case.startswith("transpose"):
            return lambda: dev.transpose(sq.deviceParams(), out.deviceParams(), 0, 1)
        return lambda: dev.tril(sq.deviceParams(), out.deviceParams(), 0)
    if case == "adam_f32":
        p, g, m, v = (_rand(dev, (1 << 16, 1024), C.F32, s) for s in range(4))

        def step():
            m2 = 0.9 * m + 0.1 * g
            v2 = 0.999 * v * v + 0.001 * g * g
            return p - (0.001 * (m2 / 0.1) / ((v2 / 0.001).sqrt() + 1e-8)), m2, v2
        return step
    raise SystemExit(f"unknown case {case}")


def run_dp_machinery(steps=30):
    """What the data-parallel forms of the MLP step cost WITHOUT any communication: one GPU, a communicator of one rank (its
    collectives move nothing), the front end told that there are two ranks. The difference to the plain step is GPU work of
    the exchange's machinery itself - scaling passes, per-parameter optimizer kernels that no longer merge, weights whose
    maximum no producer leaves - not NVLink time and not contention with a collective's kernel."""
    dev = DeviceB200(0)
    dev.commInit(0, 1, DeviceB200.commUniqueId())
    forms = {"sharded optimizer": dict(sharded=True), "sharded, deferred": dict(sharded=True, deferred=True),
             "all-reduce inside backward": dict(), "all-reduce after backward": dict(overlap=False)}
    for name, kw in forms.items():
        r = measure_mlp(dev, 1.0, steps=steps, warmup=3, rank=0, world_size=2, **kw)
        print(f"{name}: {r['ms_per_step']:.3f} ms per step, host {r['host_issue_ms_per_step']:.3f} ms, {r['kernel_launches_per_step']:.0f} launches")
    r = measure_mlp(dev, 1.0, steps=steps, warmup=3)
    print(f"plain step: {r['ms_per_step']:.3f} ms per step, host {r['host_issue_ms_per_step']:.3f} ms, {r['kernel_launches_per_step']:.0f} launches")
    dev.commDestroy()
    dev.close()


def run_case(argv):
    case = argv[0] if argv else "chain_f32"
    repeats = int(argv[1]) if len(argv) > 1 else 4
    if case == "mlp_f32_dp_machinery":
        return run_dp_machinery(repeats if len(argv) > 1 else 30)
    dev = DeviceB200(0)
    fn = build_case(dev, case)
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


# ---- bandwidth sweep of the fused chain (configuration 4) -----------------------------------------------------------------
PATTERN = 1 << 20


def tiled(dev, pattern: TensorValue, repeats: int) -> TensorValue:
    if repeats == 1:
        return pattern.reshape((1, PATTERN))
    return pattern.reshape((1, PATTERN)).broadcastTo((repeats, PATTERN)).contiguous()


def sweep_point(dev, log2n, dtype, iters=10):
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


def run_sweep(dev, max_log2n=31, min_log2n=20, dtypes=(C.F32, C.BF16)):
    out = []
    for dtype in dtypes:
        for log2n in range(min_log2n, max_log2n + 1):
            if (4 + 13) * (1 << log2n) * C.DTYPE_SIZES[dtype] > 150 * (1 << 30):
                continue                     # would not fit next to the dead intermediates of one evaluation
            out.append(sweep_point(dev, log2n, dtype, iters=10 if log2n < 28 else 5))
    return out


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "sweep":
        hi = int(sys.argv[2]) if len(sys.argv) > 2 else 31
        lo = int(sys.argv[3]) if len(sys.argv) > 3 else 20
        device = DeviceB200(0)
        for rec in run_sweep(device, hi, lo):
            print(json.dumps(rec), flush=True)
        device.close()
    else:
        run_case(sys.argv[1:])
