#!/usr/bin/env python
"""Benchmark of the B200 device on the fused elementwise chain (the headline metric), with the other kernel classes
reported beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--log2n L] [--dtype f32|bf16]

A step is one evaluation of  z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c));  s = z.sum()  over n = 2**L
elements per GPU (synthetic U(-1,1) inputs, seed 0), issued op by op through the C ABI exactly as the AIX core would
issue it: 16 recorded device calls that the device fuses into one generated kernel, plus the sum kernel.
The line also carries `mlp_train` (steps/s of the data-parallel MLP configuration at this N) and, at N = 1, `extras`
(reductions at 8192^2 bf16, matmul 4096^3) and `cpu_baseline`.
`value` counts the algorithmic bytes of the step (a, b, c read and z written once: 16*n for f32; the sum is folded into the
chain's kernel and moves nothing of its own) over the device time of K steps with inputs resident in HBM; `e2e` is the same step with the inputs copied from
pinned host memory and the sum read back every step. Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DT = {"f32": 1, "bf16": 3}
# DRAM traffic of the generated chain kernel per element, from ncu captures at n = 2^26: 1054.9 MB for f32 (algorithmic: 16
# bytes per element), 515.3 MB for bf16 (algorithmic: 8).
TRAFFIC_BYTES_PER_ELEMENT = {"f32": 1054.9e6 / (1 << 26), "bf16": 515.3e6 / (1 << 26)}
# Algorithmic bytes of one step (chain + sum) per element, both arms: a, b, c are read and z is written once; the sum needs
# no traffic of its own (the device folds it into the chain's kernel; an implementation that re-reads z is simply slower).
STEP_BYTES_PER_ELEMENT_F32 = 16.0


def chain(a, b, c, scalar_like):
    one = lambda t: scalar_like(1.0, t)
    return (a * b + c) * (one(a) / (one(a) + (-a).exp())) - b.tanh() / (one(c) + (-c).exp())


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, enabled=True):
        self.index, self.rows, self.proc, self.enabled = index, [], None, enabled
        self.begin = self.end = None

    def wait_ready(self, timeout=8.0):
        """Blocks until nvidia-smi has delivered its first sample: its start-up attaches to every GPU of the box under
        driver-wide locks (measured: a kernel launch issued during it waited 90-110 ms)."""
        t0 = time.time()
        while self.proc is not None and not self.rows and time.time() - t0 < timeout and self.proc.poll() is None:
            time.sleep(0.02)
        time.sleep(0.05)

    def mark_begin(self): self.begin = time.time()
    def mark_end(self): self.end = time.time()

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.time()] + [f.strip() for f in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        rows = self.rows
        if self.begin is not None and self.end is not None:
            inside = [r for r in rows if self.begin - 0.15 <= r[0] <= self.end + 0.15]
            rows = inside or rows            # a timed region shorter than the sampling period: fall back to all samples under load
        for r in (x[1:] for x in rows):
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def cpu_reference_chain(n_sample, repeats=1):
    """Times the reference's own front end + CPU device on n_sample elements. Returns (GB/s of algorithmic bytes, seconds)."""
    from oracle.ref_device import DeviceRefCPU
    ref = DeviceRefCPU()
    rng = np.random.default_rng(0)
    rows = max(1, n_sample // 1024)
    a, b, c = (rng.uniform(-1, 1, (rows, 1024)).astype(np.float32) for _ in range(3))
    best = None
    for _ in range(repeats):
        _, _, secs = ref.chain_f32(a, b, c)
        best = secs if best is None else min(best, secs)
    return STEP_BYTES_PER_ELEMENT_F32 * rows * 1024 / best / 1e9, best


def cpp_front_end(dev):
    """The drop-in path proper: the reference's unmodified C++ front end on aix::DeviceB200 (managed memory), timed by the
    program tests/cpp/adapter_bench.cpp. The binary is built from the reference's headers where they are present and
    travels with the repository; without it the entry says so."""
    binary = os.path.join(ROOT, "oracle", "_ref", "adapter_bench")
    if not os.path.isfile(binary):
        return {"unavailable": "adapter_bench was not built (the reference's headers were absent at build time)"}
    dev.emptyCache()
    try:
        run = subprocess.run([binary], capture_output=True, text=True, timeout=600)
        last = [l for l in run.stdout.splitlines() if l.startswith("{")]
        if run.returncode != 0 or not last:
            return {"error": (run.stdout + run.stderr)[-400:]}
        return json.loads(last[-1])
    except Exception as exc:
        return {"error": str(exc)}


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU implementation of the same step on the host cores (single-threaded: the
    reference has no threading), each step a bounded sample of the workload."""
    if rank != 0:
        return
    n_sample = 1 << 22
    from oracle.ref_device import DeviceRefCPU
    ref = DeviceRefCPU()
    rng = np.random.default_rng(0)
    a, b, c = (rng.uniform(-1, 1, (n_sample // 1024, 1024)).astype(np.float32) for _ in range(3))
    for _ in range(args.warmup):
        ref.chain_f32(a, b, c)
    total = 0.0
    for _ in range(args.steps):
        total += ref.chain_f32(a, b, c)[2]
    gbs = STEP_BYTES_PER_ELEMENT_F32 * n_sample * args.steps / total / 1e9
    line = {
        "impl": "reference", "metric": "fused-elementwise HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"fused chain + sum, f32, n=2^{args.log2n} per GPU (config 4 of the sweep)",
                   "sample": f"2^22 elements per step on the CPU"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "reference",
                         "sample": "aix::Tensor front end + aix::DeviceCPU, 2^22-element sample per step, 1 thread "
                                   f"(the reference CPU device is single-threaded) of {os.cpu_count()} host cores"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def emit(line):
    """Prints the JSON line on the real stdout (libraries such as NCCL write banners to fd 1, which main() points at
    stderr for the duration of the run)."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = os.dup(1)


def main():
    sys.stdout.flush()
    os.dup2(2, 1)                        # anything a library prints goes to stderr; the JSON line goes to _REAL_STDOUT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--log2n", type=int, default=28)
    ap.add_argument("--dtype", default="f32", choices=list(DT))
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary kernel-class measurements")
    ap.add_argument("--no-mlp", action="store_true", help="skip the MLP training measurement")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    from aix_b200 import DeviceB200, TensorValue, scalar_like, to_storage
    dev = DeviceB200(local)
    dtype = DT[args.dtype]
    esize = 4 if dtype == 1 else 2
    n = 1 << args.log2n
    rows = n // 1024
    rng = np.random.default_rng(rank)
    host = [to_storage(rng.uniform(-1, 1, n).astype(np.float32), dtype) for _ in range(3)]
    pinned = []
    for h in host:                           # pinned host copies for the end-to-end leg
        t = torch.from_numpy(h.view(np.int16) if dtype == 3 else h).pin_memory()
        pinned.append(t)
    a, b, c = (TensorValue.empty((rows, 1024), dev, dtype) for _ in range(3))
    for t, p in zip((a, b, c), pinned):
        dev.copy(p.data_ptr(), dtype, t.storage.data, dtype, n)
    dev.synchronize()

    def step():
        z = chain(a, b, c, scalar_like)
        return z, z.sum()

    # One clock sampler, on rank 0 only, started before anything is timed and waited for until its first sample has
    # arrived: nvidia-smi takes driver-wide locks while it starts (measured: a launch that fell into that window waited
    # ~100 ms, inside 7 ms of timed work). It keeps sampling through the warm-up (same kernels, same load) and the timed
    # region; the summary prefers the samples that fall inside the timed region.
    clocks = ClockSampler(local, enabled=(rank == 0))
    clocks.__enter__()
    clocks.wait_ready()
    warm0 = dev.stats()
    warm_marker = dev.createEvent()
    for _ in range(args.warmup):
        z, s = step()
        dev.recordEvent(warm_marker)     # flush per step, exactly as in the timed loop: the recorder would otherwise merge the
                                         # warm-up steps into one differently shaped kernel and leave the real one uncompiled
    dev.synchronize()
    # The device folds z.sum() into the chain's kernel when it is recorded behind it (one launch per step, z is still
    # written: 16 bytes per element); with that switched off the sum is a second kernel that reads z again (20 bytes).
    sum_fused = dev.stats()["reductions_fused"] - warm0["reductions_fused"] >= args.warmup > 0
    del z, s

    # ---- timed region: K steps, device time, max over ranks ------------------------------------------------------
    ev0, ev1 = dev.createEvent(), dev.createEvent()
    kev = [(dev.createEvent(), dev.createEvent()) for _ in range(args.steps)]
    stats0 = dev.stats()
    barrier()
    dev.synchronize()
    clocks.mark_begin()
    dev.recordEvent(ev0)
    for k in range(args.steps):
        dev.recordEvent(kev[k][0])
        z = chain(a, b, c, scalar_like)
        if sum_fused:
            s = z.sum()                      # recorded behind the chain: same kernel
        dev.recordEvent(kev[k][1])           # flushes: the fused chain kernel runs between the two events
        if not sum_fused:
            s = z.sum()
    dev.recordEvent(ev1)
    dev.synchronize()
    clocks.mark_end()
    barrier()
    clocks.__exit__(None, None, None)
    stats1 = dev.stats()
    ms_total = max_over_ranks(dev.elapsedMs(ev0, ev1))
    launch_ms = [float(dev.elapsedMs(x, y)) for x, y in kev]
    chain_ms = float(np.mean(launch_ms))           # the average launch duration over the timed region
    result_sum = float(s.item())
    step_bytes = 4 * n * esize        # algorithmic bytes of one step, whether or not the sum runs as a kernel of its own
    value = world * step_bytes * args.steps / (ms_total * 1e-3) / 1e9
    launches = stats1["total_kernel_launches"] - stats0["total_kernel_launches"]

    # ---- end to end: inputs from pinned host memory every step, sum read back every step --------------------------
    e2e_steps = max(2, min(args.steps, 5))
    for p, t in zip(pinned, (a, b, c)):
        dev.copy(p.data_ptr(), dtype, t.storage.data, dtype, n)
    dev.synchronize()
    barrier()
    t0 = time.perf_counter()
    dev.recordEvent(ev0)
    for _ in range(e2e_steps):
        for p, t in zip(pinned, (a, b, c)):
            dev.copy(p.data_ptr(), dtype, t.storage.data, dtype, n)
        z, s = step()
        _ = s.item()                             # device -> host read of the step's result
    dev.recordEvent(ev1)
    dev.synchronize()
    e2e_ms = max_over_ranks(max(dev.elapsedMs(ev0, ev1), 1e3 * (time.perf_counter() - t0)))
    e2e_value = world * step_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
    del z, s

    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    chain_bytes = 4 * n * esize
    achieved = chain_bytes / (chain_ms * 1e-3) / 1e9
    line = {
        "metric": "fused-elementwise HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"fused chain z=(a*b+c)*sigmoid(a)-tanh(b)/(1+exp(-c)) + z.sum(), {args.dtype}, n=2^{args.log2n} "
                               f"elements per GPU as [{rows},1024] (config 4 of the sweep; config 0 expression)",
                   "l2": f"inputs are {3 * n * esize >> 20} MiB per step, larger than the 126 MB L2; no explicit flush",
                   "sharding": "rows split across ranks, no data-path collective", "bytes_per_step_per_gpu": step_bytes,
                   "bytes_counted": "a, b, c read + z written once per step; z.sum() " +
                                    ("is folded into the chain kernel" if sum_fused else "runs as a second kernel that re-reads z (not counted)")},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 3 * n * esize, "d2h_bytes_per_step": esize,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": TRAFFIC_BYTES_PER_ELEMENT.get(args.dtype, 0) * n or None,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of this kernel captured at n=2^26, scaled by n "
                                       "(traffic is proportional to n)",
                     "kernel": "generated fused chain kernel" + (" with the sum folded in as a reduction epilogue" if sum_fused else ""),
                     "bytes_per_launch": chain_bytes,
                     "ms_per_launch": chain_ms, "ms_per_launch_median": float(np.median(launch_ms)),
                     "ms_each_launch": [round(x, 4) for x in launch_ms[:32]],
                     "peak_kind": f"of {peak_kind}", "frac_of_8tbs_nominal": achieved / 8000.0},
        "checksum": result_sum,
        "fusion": {k: stats1[k] - stats0[k] for k in ("ops_recorded", "fused_kernels", "fused_ops", "fills_absorbed", "stores_elided",
                                                      "reductions_fused", "kernel_cache_hits", "kernel_cache_misses")},
    }

    # ---- the data-parallel MLP training configuration, at every N (gradient exchange over NCCL for N > 1) ----------------
    mlp_train = None
    if not args.no_mlp:
        # free the sweep tensors first: the MLP step needs its own few GB
        del a, b, c
        dev.emptyCache()
        try:
            if world > 1:
                ids = [DeviceB200.commUniqueId() if rank == 0 else None]
                dist.broadcast_object_list(ids, src=0)
                dev.commInit(rank, world, ids[0])
            from bench_cases import measure_mlp
            mlp_steps = 100                              # the configuration is "100 steps from seed 0"
            common = dict(steps=mlp_steps, warmup=3, rank=rank, world_size=world, barrier=barrier, reduce_max=max_over_ranks)
            if world == 1:
                mlp_train = measure_mlp(dev, tensor_peak, **common)
            else:
                # default form: sharded optimizer (reduce-scatter, 1/N of Adam per rank, all-gather on a communicator of its own);
                # beside it the two all-reduce forms and the optional forms of the sharded optimizer (late layers' updates deferred
                # into the next forward pass, early layers' moved into backward), to show what each step of the design buys
                mlp_train = measure_mlp(dev, tensor_peak, sharded=True, **common)
                inside = measure_mlp(dev, tensor_peak, **common)
                mlp_train["ms_per_step_all_reduce_inside_backward"] = inside["ms_per_step"]
                mlp_train["host_issue_ms_per_step_all_reduce_inside_backward"] = inside["host_issue_ms_per_step"]
                mlp_train["ms_per_step_all_reduce_after_backward"] = measure_mlp(dev, tensor_peak, overlap=False, **common)["ms_per_step"]
                mlp_train["ms_per_step_deferred"] = measure_mlp(dev, tensor_peak, sharded=True, deferred=True, **common)["ms_per_step"]
                mlp_train["ms_per_step_deferred_early"] = measure_mlp(dev, tensor_peak, sharded=True, deferred=True, early=True, **common)["ms_per_step"]
                # ... and the sharded optimizer with every collective on ONE communicator (read when the communicator is created,
                # hence a second one)
                try:
                    dev.commDestroy()
                    os.environ["AIXB200_COMM_GATHER_LANE"] = "0"
                    ids = [DeviceB200.commUniqueId() if rank == 0 else None]
                    dist.broadcast_object_list(ids, src=0)
                    dev.commInit(rank, world, ids[0])
                    measure_mlp(dev, tensor_peak, sharded=True, **dict(common, steps=5))      # the new communicator sets up its connections
                    mlp_train["ms_per_step_one_communicator"] = measure_mlp(dev, tensor_peak, sharded=True, **common)["ms_per_step"]
                except Exception as exc:
                    mlp_train["one_communicator_error"] = str(exc)
                finally:
                    os.environ.pop("AIXB200_COMM_GATHER_LANE", None)
                # the broadcast + reduction configuration with its rows split over the ranks (one scalar all-reduce for the mean)
                from bench_cases import measure_config1_sharded
                line["config1_sharded"] = measure_config1_sharded(dev, hbm_peak, rank, world, barrier=barrier, reduce_max=max_over_ranks)
                means = [None] * world
                dist.all_gather_object(means, line["config1_sharded"]["local_mean_of_this_rank"])
                line["config1_sharded"]["mean_of_local_means"] = float(np.mean(means))
                dev.commDestroy()
        except Exception as exc:
            mlp_train = {"error": str(exc)}

    if rank == 0 and world == 1:
        try:
            gbs, secs = cpu_reference_chain(1 << 25)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "reference",
                                    "sample": f"aix::Tensor front end + aix::DeviceCPU on 2^25 elements ({secs:.1f} s), 1 thread of "
                                              f"{os.cpu_count()} host cores (the reference CPU device is single-threaded)"}
        except Exception as exc:                  # the oracle library is test infrastructure; report, do not hide
            line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 1, "kind": "reference", "sample": f"unavailable: {exc}"}
        if not args.no_extras:
            try:
                from bench_cases import measure_extras
                line["extras"] = measure_extras(dev, hbm_peak, tensor_peak)
            except Exception as exc:
                line["extras"] = {"error": str(exc)}
            line["extras"]["cpp_front_end"] = cpp_front_end(dev)
    if mlp_train is not None:
        line["mlp_train"] = mlp_train                    # last key: the step time of this N stays in the tail of the line
    if rank == 0:
        emit(line)
    dev.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
