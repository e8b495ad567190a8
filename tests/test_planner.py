"""Host logic of the lazy recorder, fusion planner, code generator and allocator on a dry-run device: ops are
recorded, planned and compiled with NVRTC for sm_100a, but nothing is launched (no GPU needed).
Modelled on the reference's FuseEngine unit tests with fake back ends (Targets/AIXTests/DeviceTests.cpp:235-289,
1810-1879)."""
import numpy as np
import pytest

from aix_b200 import BF16, F16, F32, I32, DeviceB200, TensorValue, scalar_like


def delta(dev, before):
    after = dev.stats()
    return {k: after[k] - before[k] for k in after}


def chain(a, b, c):
    one = lambda t: scalar_like(1.0, t)
    return (a * b + c) * (one(a) / (one(a) + (-a).exp())) - b.tanh() / (one(c) + (-c).exp())


def test_chain_becomes_one_kernel_with_one_store(dry):
    a, b, c = (TensorValue.full(0.5, (64, 64), dry) for _ in range(3))
    dry.synchronize()
    s0 = dry.stats()
    z = chain(a, b, c)
    dry.synchronize()
    d = delta(dry, s0)
    assert d["ops_recorded"] == 16 and d["fused_kernels"] == 1 and d["fused_ops"] == 13
    assert d["fills_absorbed"] == 3 and d["stores_elided"] == 12
    src = dry.lastKernelSource()
    assert src.count("*(Pack<Df32::S, 4>*)(s0") == 1 and "s1" not in src.split("extern")[1]      # z is the only store
    assert "Pack<Df32::S, 4>*)(l2" in src                                                         # 128-bit loads


def test_live_intermediates_are_written(dry):
    a, b = TensorValue.full(1.0, (1000,), dry), TensorValue.full(2.0, (1000,), dry)
    dry.synchronize()
    s0 = dry.stats()
    t = a * b            # kept alive by the caller: must reach memory
    u = t + a
    dry.synchronize()
    d = delta(dry, s0)
    assert d["fused_kernels"] == 1 and d["stores_elided"] == 0


def test_scalar_values_do_not_change_the_kernel(dry):
    x = TensorValue.full(1.0, (8, 8), dry)
    dry.synchronize()
    y1 = x * 2.0 + 1.0
    dry.synchronize()
    s0 = dry.stats()
    y2 = x * 3.0 + 5.0
    dry.synchronize()
    d = delta(dry, s0)
    assert d["kernel_cache_misses"] == 0 and d["kernel_cache_hits"] == 1 and d["fills_absorbed"] == 2


def test_different_sizes_go_to_different_kernels_but_interleaved_chains_still_fuse(dry):
    a, b = TensorValue.full(1.0, (100,), dry), TensorValue.full(1.0, (200,), dry)
    dry.synchronize()
    s0 = dry.stats()
    a1 = a + 1.0
    b1 = b + 1.0
    a2 = a1 * a        # joins the first kernel although an op of another size was recorded in between
    b2 = b1 * b
    dry.synchronize()
    d = delta(dry, s0)
    assert d["fused_kernels"] == 2 and d["fused_ops"] == 6


def test_reading_a_transposed_view_of_a_pending_result_forces_a_second_kernel(dry):
    a = TensorValue.full(1.0, (16, 16), dry)
    dry.synchronize()
    s0 = dry.stats()
    t = a + 1.0
    u = t.transpose(0, 1) + a          # element i of u needs element j != i of t: needs a grid-wide barrier
    dry.synchronize()
    assert delta(dry, s0)["fused_kernels"] == 2


def test_in_place_update_stays_in_one_kernel_and_in_program_order(dry):
    m, g = TensorValue.full(1.0, (4096,), dry), TensorValue.full(2.0, (4096,), dry)
    dry.synchronize()
    s0 = dry.stats()
    m *= 0.9
    m += 0.1 * g
    out = m / 0.5
    dry.synchronize()
    d = delta(dry, s0)
    assert d["fused_kernels"] == 1
    body = dry.lastKernelSource().split("extern")[1]
    assert body.count("*)(s") == 2          # m (its final value only) and out


def test_broadcast_operands_use_hoisted_index_paths(dry):
    x = TensorValue.full(1.0, (64, 128), dry)
    row, col = TensorValue.full(1.0, (128,), dry), TensorValue.full(1.0, (64, 1), dry)
    y = x * row + col
    dry.synchronize()
    src = dry.lastKernelSource()
    assert "packs per row" in src and "qt" in src          # row vector: running column; column vector: running row
    assert " % cp" in src.split("for (; pk < nvec")[0]      # the modulo sits before the loop, not inside it


def test_sixteen_bit_chains_use_packed_arithmetic(dry):
    for dt, name in ((BF16, "bf16x2"), (F16, "f16x2")):
        a, b = TensorValue.full(1.0, (64, 64), dry, dt), TensorValue.full(1.0, (64, 64), dry, dt)
        z = (a * b + a).tanh()
        dry.synchronize()
        body = dry.lastKernelSource().split("extern")[1]
        assert "pp_mul" in body and "pp_tanh" in body and f"add.rn.{name}" in dry.lastKernelSource()


def test_all_element_types_generate_compilable_kernels(dry):
    for dt in range(9):
        a = TensorValue.full(3.0, (33,), dry, dt)
        b = TensorValue.full(2.0, (33,), dry, dt)
        r = (a + b) * a - b
        r = r / b
        q = TensorValue.empty(r.shape, dry, dt)
        for op in ("sqrt", "sin", "cos", "tanh", "log", "exp"):
            getattr(dry, op)(r.deviceParams(), q.deviceParams())
        dry.pow(r.deviceParams(), b.deviceParams(), q.deviceParams())
        c = r.to((dt + 3) % 9)
        dry.synchronize()                   # NVRTC would fail here on bad generated code


def test_flush_threshold_and_statistics(dry):
    x = TensorValue.full(1.0, (256,), dry)
    one = TensorValue.full(1.0, (256,), dry)
    dry.synchronize()
    s0 = dry.stats()
    for _ in range(450):
        x += one
    d = delta(dry, s0)
    assert d["flushes"] == 2 and d["ops_recorded"] == 450        # two automatic flushes at 200 pending ops
    dry.synchronize()


def test_allocator_reuses_blocks_and_defers_frees_until_the_flush(dry):
    dry.synchronize()
    dry.emptyCache()
    s0 = dry.stats()
    a = TensorValue.full(1.0, (1 << 16,), dry)
    for _ in range(5):
        t = a + 1.0
        del t                       # dead before the flush: its block must not be handed out again while pending
        dry.synchronize()
    d = delta(dry, s0)
    assert d["cuda_mallocs"] <= 4           # a, one scalar-fill temporary, one result block: reused afterwards
    assert dry.stats()["bytes_cached"] > 0
    dry.emptyCache()
    assert dry.stats()["bytes_cached"] == 0


def test_fusion_can_be_switched_off():
    dev = DeviceB200(0, dry_run=1, disk_cache=0, fusion=0)
    a = TensorValue.full(1.0, (64,), dev)
    dev.synchronize()
    s0 = dev.stats()
    z = (a + 1.0) * a
    dev.synchronize()
    d = delta(dev, s0)
    assert d["fused_kernels"] == 3          # fill, add, mul: one kernel each
    dev.close()


def test_full_reductions_join_the_kernel_that_produces_their_operand(dry):
    a, b = TensorValue.full(1.0, (64, 1024), dry), TensorValue.full(2.0, (64, 1024), dry)
    dry.synchronize()
    s0 = dry.stats()
    d = a - b
    loss = (d * d).sum()                  # the product is dead: neither d*d nor (once d dies) d needs memory
    peak = (a * b).max()
    del d
    mean = loss / 65536.0                 # reads the reduction's result: next kernel
    dry.synchronize()
    st = delta(dry, s0)
    assert st["reductions_fused"] == 2 and st["fused_kernels"] == 2 and st["static_kernel_launches"] == 0
    assert st["stores_elided"] >= 3
    first, second = None, dry.lastKernelSource()
    assert "red_finish" not in second.split("extern")[1]             # the division kernel has no reduction


def test_reduction_kernel_source_has_one_epilogue_per_reduction(dry):
    a = TensorValue.full(1.0, (1000,), dry)
    dry.synchronize()
    t = a * 3.0
    s, m = t.sum(), t.max()
    dry.synchronize()
    body = dry.lastKernelSource().split("extern")[1]
    assert body.count("red_finish<Red<Df32, false> >") == 1 and body.count("red_finish<Red<Df32, true> >") == 1
    assert "racc0 = Red<Df32, false>::step" in body and "racc1 = Red<Df32, true>::step" in body


def test_reduction_of_a_tensor_already_in_memory_is_not_recorded(dry):
    a = TensorValue.full(1.0, (1000,), dry)
    dry.synchronize()
    s0 = dry.stats()
    s = a.sum()
    dry.synchronize()
    st = delta(dry, s0)
    assert st["reductions_fused"] == 0 and st["fused_kernels"] == 0


def test_result_of_a_reduction_orders_later_writers_and_readers(dry):
    a = TensorValue.full(2.0, (4096,), dry)
    dry.synchronize()
    s0 = dry.stats()
    t = a * a
    s = t.sum()
    u = t + s.broadcastTo((4096,)) if hasattr(s, "broadcastTo") else t + t     # reads the scalar: a later kernel
    s.fill(0.0)                                                                # overwrites it: not before the reduction ran
    dry.synchronize()
    st = delta(dry, s0)
    assert st["reductions_fused"] == 1 and st["fused_kernels"] >= 2


def test_reduction_epilogue_compiles_in_unusual_kernels(dry):
    """Kernels whose only output is a reduction (no loads, or no stores), in-place updates of the reduced tensor after the
    reduction, integer and 16-bit element types: every variant must plan and compile."""
    s0 = dry.stats()
    ones = TensorValue.full(1.0, (3, 1000), dry)
    total = ones.sum()                                   # producer is a pending fill: no load, and (ones stays alive) one store
    del ones
    a = TensorValue.full(2.0, (4099,), dry, BF16)
    b = TensorValue.full(3.0, (4099,), dry, BF16)
    dry.synchronize()
    t = a * b
    s = t.sum()
    m = t.max()
    t += a                                               # in-place update after the reductions: they saw the old values
    again = t.sum()
    i = TensorValue.full(7, (513,), dry, I32)
    dry.synchronize()
    k = (i * i).max()
    j = (i + i).sum()
    dry.synchronize()
    st = delta(dry, s0)
    assert st["reductions_fused"] == 6 and st["static_kernel_launches"] == 0


def test_reduction_is_not_recorded_with_fusion_off():
    from aix_b200 import DeviceB200
    dev = DeviceB200(0, dry_run=1, disk_cache=0, fusion=0)
    a = TensorValue.full(1.0, (1000,), dev)
    s = (a * a).sum()
    dev.synchronize()
    assert dev.stats()["reductions_fused"] == 0
    dev.close()


def test_descriptors_that_alias_through_different_base_pointers_are_ordered(dry):
    """Hazards are found on byte ranges, not on the `data` pointer: a descriptor whose base is an interior pointer of a
    buffer written by a pending op must not be fused with that op as if it were independent."""
    from aix_b200 import DeviceTensorParams
    whole = TensorValue.full(1.0, (1024,), dry)
    other = TensorValue.full(2.0, (512,), dry)
    dry.synchronize()
    s0 = dry.stats()
    upper = DeviceTensorParams(whole.storage.data, F32, 512, (512,), 512, (1,))                   # elements 512 .. 1023
    dry.add(upper, other.deviceParams(), upper)                                                  # pending in-place write
    same_bytes = DeviceTensorParams(whole.storage.data + 512 * 4, F32, 0, (512,), 512, (1,))      # same bytes, other base
    out = TensorValue.empty((512,), dry)
    dry.add(same_bytes, other.deviceParams(), out.deviceParams())  # same element count: would join the writer's kernel
    dry.synchronize()
    assert delta(dry, s0)["fused_kernels"] == 2, "the aliasing read must wait for the writer's kernel"
    s1 = dry.stats()
    t = other + 1.0                                                 # reads `other` ...
    shifted = DeviceTensorParams(other.storage.data + 4, F32, 0, (511,), 511, (1,))
    dry.fill(0.0, F32, shifted)                                     # ... then part of it is overwritten through another base
    u = other * 2.0
    dry.synchronize()
    assert delta(dry, s1)["fused_kernels"] == 3, "reader, overlapping writer, reader: three kernels in program order"


def test_idle_fills_stay_recorded_until_something_uses_their_buffer(dry):
    """zeroGrad() fills every gradient, and the accumulation `grad += dW` comes several matmuls later: a fill that nothing
    else touches survives the flushes in between (the reference defers such fills too, aixFuse.cpp:891-916) and is then
    absorbed by the accumulation instead of costing a kernel and a pass over the buffer."""
    a, b = TensorValue.full(1.0, (128, 128), dry), TensorValue.full(2.0, (128, 128), dry)
    dry.synchronize()
    s0 = dry.stats()
    g = TensorValue.full(0.0, (128, 128), dry)           # idle fill
    c = a.matmul(b)                                      # flushes the recorder; the fill has nothing to do with it
    d1 = delta(dry, s0)
    assert d1["fused_kernels"] == 0, "the idle fill must not be launched by the matmul's flush"
    g += c                                               # the accumulation absorbs it: g = 0 + c in one kernel, no load of g
    dry.synchronize()
    d2 = delta(dry, s0)
    assert d2["fused_kernels"] == 1 and d2["fills_absorbed"] >= 1
    assert dry.lastKernelSource().count("const Df32::S* const l") == 1       # one load (c), not two
    # synchronize() emits whatever is still recorded: the host may read the buffer afterwards
    s1 = dry.stats()
    h = TensorValue.full(3.0, (64,), dry)
    e = a.matmul(b)
    assert delta(dry, s1)["fused_kernels"] == 0
    dry.synchronize()
    assert delta(dry, s1)["fused_kernels"] == 1
    # a call that touches the buffer itself flushes the fill first
    s2 = dry.stats()
    k = TensorValue.full(0.0, (128, 128), dry)
    dry.matmul(a.deviceParams(), b.deviceParams(), k.deviceParams())          # k is the result: its fill must not come after
    assert delta(dry, s2)["fused_kernels"] == 1
