"""Parity of sum / max / reduceTo / maxTo with the reference's CPU device (Tests/DeviceTests.cpp:560-700, 1990-2150).

Floating sums: the CPU device accumulates sequentially in the storage type, so for f32 the comparison is bounded by
1e-5 * sum(|x|) and additionally checked against the float64 sum; for f16/bf16 the oracle is the CPU device applied
to the same values widened to f32 (accumulate in f32, round once), because a 16-bit accumulator saturates.
"""
import numpy as np
import pytest

from aix_b200 import BF16, DTYPE_NAMES, F16, F32, F64, I8, I16, I32, I64, U8, TensorValue, to_storage, from_storage
from conftest import assert_close

pytestmark = pytest.mark.gpu

SIZES = [1, 2, 3, 5, 8, 17, 33, 64, 127, 255, 1025, 2049, 65537, 1 << 20]
ALL_DTYPES = [F64, F32, F16, BF16, I64, I32, I16, I8, U8]
FLOATS = [F64, F32, F16, BF16]


def values(rng, shape, dtype):
    if dtype in FLOATS:
        x = rng.normal(0, 1, shape)
        return from_storage(to_storage(x, dtype), dtype).astype(np.float64) if dtype != F64 else x
    if dtype == U8:
        return rng.integers(0, 255, shape)
    return rng.integers(-100, 100, shape)


def wide(dtype):
    return F32 if dtype in (F16, BF16) else dtype


def round_to(x, dtype):
    return from_storage(to_storage(x, dtype), dtype)


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_sum_and_max_of_everything(b200, ref, dtype):
    rng = np.random.default_rng(100 + dtype)
    for n in SIZES:
        x = values(rng, n, dtype)
        g = TensorValue.from_numpy(x, b200, dtype)
        r = TensorValue.from_numpy(x, ref, wide(dtype))
        got_sum, got_max = g.sum().numpy(), g.max().numpy()
        want_max = r.max().numpy()
        assert_close(got_max, round_to(want_max, dtype), dtype, f"max n={n}")
        if dtype in FLOATS:
            exact = np.sum(np.asarray(x, dtype=np.float64))
            bound = {F64: 1e-12, F32: 1e-5, F16: 1e-2, BF16: 1e-2}[dtype]
            assert abs(float(got_sum) - exact) <= bound * max(1.0, float(np.sum(np.abs(x)))), f"sum n={n}"
            if dtype in (F16, BF16):
                if np.isfinite(round_to(np.array([exact]), dtype)[0]):
                    assert_close(got_sum, round_to(r.sum().numpy(), dtype), dtype, f"sum n={n}", scale=max(1.0, abs(exact)))
        else:
            assert_close(got_sum, r.sum().numpy(), dtype, f"sum n={n}")


def test_sum_of_strided_views(b200, ref):
    rng = np.random.default_rng(8)
    x = rng.normal(0, 1, (63, 130)).astype(np.float32)
    for dev_pair in [(b200, ref)]:
        outs = []
        for dev in dev_pair:
            t = TensorValue.from_numpy(x, dev).transpose(0, 1)
            row = t.select(0, 5)
            outs.append((t.sum().numpy(), t.max().numpy(), row.sum().numpy(), row.max().numpy()))
        for a, b in zip(*outs):
            assert_close(a, b, F32, "strided", scale=float(np.abs(x).sum()))


SHAPES = [((7, 5), 1), ((7, 5), 0), ((64, 1024), 1), ((64, 1024), 0), ((33, 2049), 1), ((1025, 40), 0), ((4, 5, 6), 1),
          ((4, 5, 6), 0), ((4, 5, 6), 2), ((300, 8192), 1), ((4096, 96), 0), ((2, 3, 4, 5), 2)]


@pytest.mark.parametrize("dtype", [F32, F64, BF16, F16, I32, I8, U8, I64, I16], ids=lambda d: DTYPE_NAMES[d])
def test_reduce_to_and_max_to_along_one_dimension(b200, ref, dtype):
    rng = np.random.default_rng(200 + dtype)
    for shape, dim in SHAPES:
        x = values(rng, shape, dtype)
        g = TensorValue.from_numpy(x, b200, dtype)
        r = TensorValue.from_numpy(x, ref, wide(dtype))
        got_sum, got_max = g.sum(dim).numpy(), g.max(dim).numpy()
        want_sum, want_max = r.sum(dim).numpy(), r.max(dim).numpy()
        assert_close(got_max, round_to(want_max, dtype), dtype, f"maxTo {shape} dim {dim}")
        scale = np.maximum(1.0, np.abs(np.asarray(x, dtype=np.float64)).sum(axis=dim)) if dtype in FLOATS else None
        assert_close(got_sum, round_to(want_sum, dtype) if dtype in FLOATS else want_sum, dtype, f"reduceTo {shape} dim {dim}", scale=scale)


def test_reduce_to_broadcast_shapes(b200, ref):
    """reduceTo as the backward of broadcasting: arbitrary target shapes incl. lower rank (aixCore.hpp:2029-2036)."""
    rng = np.random.default_rng(9)
    cases = [((6, 4, 5), (4, 5)), ((6, 4, 5), (5,)), ((6, 4, 5), (1, 4, 1)), ((6, 4, 5), (6, 1, 5)), ((6, 4, 5), (1,)),
             ((6, 4, 5), ()), ((128, 256), (1, 256)), ((128, 256), (256,)), ((128, 256), (128, 1))]
    for src_shape, dst_shape in cases:
        x = rng.normal(0, 1, src_shape).astype(np.float32)
        outs = []
        for dev in (b200, ref):
            outs.append(TensorValue.from_numpy(x, dev).reduceTo(dst_shape).numpy())
        assert_close(outs[0], outs[1], F32, f"reduceTo {src_shape} -> {dst_shape}", scale=max(1.0, float(np.abs(x).sum()) / max(1, outs[1].size)))


def test_reduce_to_accumulates_into_destination(b200, ref):
    """The device contract is dst += sum(src): a destination that is not zero keeps its contents."""
    rng = np.random.default_rng(10)
    x = rng.normal(0, 1, (50, 70)).astype(np.float32)
    outs = []
    for dev in (b200, ref):
        t = TensorValue.from_numpy(x, dev)
        dst = TensorValue.full(5.0, (1, 70), dev)
        dev.reduceTo(t.deviceParams(), dst.deviceParams())
        mx = TensorValue.full(0.5, (50, 1), dev)
        dev.maxTo(t.deviceParams(), mx.deviceParams())
        outs.append((dst.numpy(), mx.numpy()))
    assert_close(outs[0][0], outs[1][0], F32, "reduceTo accumulate", scale=50.0)
    assert_close(outs[0][1], outs[1][1], F32, "maxTo accumulate")


def relu(v):
    """relu composed from device ops, identically on every device: (v + sqrt(v*v)) * 0.5."""
    return (v + (v * v).sqrt()) * 0.5


def config1(dev, x, g, bias, dtype):
    tx, tg, tb = (TensorValue.from_numpy(v, dev, dtype) for v in (x, g, bias))
    y = relu(tx * tg + tb)
    return y, y.sum(1), y.max(1), y.mean()


@pytest.mark.parametrize("rows,cols", [(256, 512), (1000, 1000)])
def test_config1_broadcast_and_reductions_bf16(b200, ref, rows, cols):
    """y = relu(x*g + bias) in bf16; row sums, row maxima and the global mean accumulate in f32."""
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (rows, cols)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    bias = rng.normal(0, 0.1, cols).astype(np.float32)
    gy, gsum, gmax, gmean = config1(b200, x, g, bias, BF16)
    ry, _, rmax, _ = config1(ref, x, g, bias, BF16)
    y_ref = ry.numpy()
    assert_close(gy.numpy(), y_ref, BF16, "y")
    assert_close(gmax.numpy(), rmax.numpy(), BF16, "row max")
    # 16-bit reductions: oracle = CPU device on the f32-widened y, rounded once to bf16
    wide_y = TensorValue.from_numpy(y_ref, ref, F32)
    assert_close(gsum.numpy(), round_to(wide_y.sum(1).numpy(), BF16), BF16, "row sum", scale=np.maximum(1.0, y_ref.sum(axis=1)))
    want_mean = round_to(np.array(round_to(np.array(y_ref.astype(np.float64).sum()), BF16) / round_to(np.array(float(y_ref.size)), BF16)), BF16)
    assert_close(gmean.numpy(), want_mean, BF16, "mean")


# ---- full reductions folded into the producing kernel ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_sum_and_max_fused_behind_their_producer(b200, ref, dtype):
    """`(a op b).sum()` / `.max()` with the elementwise op still pending: the reduction runs as an epilogue of the generated
    kernel. Oracle as above: the CPU device on the same op sequence (16-bit floats: elementwise in the 16-bit type,
    reduction on the values widened to f32)."""
    rng = np.random.default_rng(300 + dtype)
    for n in [2, 3, 5, 17, 127, 1025, 2049, 65537, (1 << 20) + 3]:
        x, y = values(rng, n, dtype), values(rng, n, dtype)
        before = b200.stats()["reductions_fused"]
        ga, gb = TensorValue.from_numpy(x, b200, dtype), TensorValue.from_numpy(y, b200, dtype)
        b200.synchronize()
        kept = ga + gb                                  # stays alive: stored AND reduced
        got_sum, got_max = kept.sum(), kept.max()
        got_dead = (ga * gb).sum()                      # the product never reaches memory
        got_sum, got_max, got_dead, got_kept = got_sum.numpy(), got_max.numpy(), got_dead.numpy(), kept.numpy()
        assert b200.stats()["reductions_fused"] - before == 3, "the reductions were not folded into the producer's kernel"

        ra, rb = TensorValue.from_numpy(x, ref, dtype), TensorValue.from_numpy(y, ref, dtype)
        rkept, rprod = ra + rb, ra * rb
        assert_close(got_kept, rkept.numpy(), dtype, f"kept n={n}")
        want_max = rkept.max().numpy()
        assert_close(got_max, want_max, dtype, f"max n={n}")
        if dtype in FLOATS:
            for got, r in ((got_sum, rkept), (got_dead, rprod)):
                vals = np.asarray(r.numpy(), dtype=np.float64)
                exact = vals.sum()
                bound = {F64: 1e-12, F32: 1e-5, F16: 1e-2, BF16: 1e-2}[dtype]
                assert abs(float(got) - exact) <= bound * max(1.0, float(np.abs(vals).sum())), f"sum n={n}"
                if dtype in (F16, BF16) and np.isfinite(round_to(np.array([exact]), dtype)[0]):
                    assert_close(got, round_to(r.to(F32).sum().numpy(), dtype), dtype, f"sum n={n}", scale=max(1.0, abs(exact)))
        else:
            assert_close(got_sum, rkept.sum().numpy(), dtype, f"sum n={n}")
            assert_close(got_dead, rprod.sum().numpy(), dtype, f"dead sum n={n}")


def test_fused_reduction_result_feeds_later_ops_and_repeats_exactly(b200, ref):
    rng = np.random.default_rng(9)
    x = rng.normal(0, 1, (1 << 18,)).astype(np.float32)
    t = rng.normal(0, 1, (1 << 18,)).astype(np.float32)
    outs = []
    for dev in (b200, ref):
        p, q = TensorValue.from_numpy(x, dev), TensorValue.from_numpy(t, dev)
        dev.synchronize()
        diff = p - q
        loss = (diff * diff).sum() / float(x.size)      # mean squared error: sum folded, division in the next kernel
        again = ((p - q) * (p - q)).sum() / float(x.size)
        outs.append((loss.numpy(), again.numpy()))
    assert np.array_equal(outs[0][0], outs[0][1]), "same grid, same fold order: bit-identical repeats"
    # the CPU device sums 2^18 values sequentially in f32 (itself ~1e-4 off): both are held against the float64 value
    exact = float(np.mean(np.square((x - t).astype(np.float32).astype(np.float64))))
    assert abs(float(outs[0][0]) - exact) <= 1e-5 * exact, (outs[0][0], exact)
    assert abs(float(outs[1][0]) - exact) <= 5e-4 * exact, (outs[1][0], exact)


def test_fused_reduction_over_a_broadcast_chain_bf16(b200, ref):
    rng = np.random.default_rng(10)
    x = rng.normal(0, 1, (512, 1024)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, (1024,)).astype(np.float32)
    res = []
    for dev in (b200, ref):
        tx, tg = TensorValue.from_numpy(x, dev, BF16), TensorValue.from_numpy(g, dev, BF16)
        dev.synchronize()
        v = tx * tg
        y = (v + (v * v).sqrt()) * 0.5
        if dev is b200:
            res.append((y.sum().numpy(), y.max().numpy()))
        else:
            res.append((round_to(y.to(F32).sum().numpy(), BF16), y.max().numpy()))
    assert_close(res[0][1], res[1][1], BF16, "max")
    assert_close(res[0][0], res[1][0], BF16, "sum", scale=float(abs(res[1][0])))


def test_fused_reduction_sees_the_values_at_its_place_in_program_order(b200, ref):
    """A reduction folded into a kernel reads the producer's register at the point where it was recorded: a later in-place
    update of the same tensor inside the same kernel must not leak into it. Also: a pending fill as the producer."""
    rng = np.random.default_rng(12)
    x = rng.normal(0, 1, (3, 4099)).astype(np.float32)
    y = rng.normal(0, 1, (3, 4099)).astype(np.float32)
    got, want = [], []
    for dev, out in ((b200, got), (ref, want)):
        a, b = TensorValue.from_numpy(x, dev), TensorValue.from_numpy(y, dev)
        dev.synchronize()
        t = a * b
        before, peak = t.sum(), t.max()
        t += a                                  # same storage, same kernel on the B200
        after = t.sum()
        ones = TensorValue.full(0.5, (7, 1000), dev)
        out.extend([before.numpy(), peak.numpy(), after.numpy(), t.numpy(), ones.sum().numpy()])
    scale = float(np.abs(x * y).sum())
    assert_close(got[0], want[0], F32, "sum before the update", scale=scale)
    assert_close(got[1], want[1], F32, "max before the update")
    assert_close(got[2], want[2], F32, "sum after the update", scale=scale)
    assert_close(got[3], want[3], F32, "updated tensor")
    assert float(got[4]) == 3500.0 == float(want[4])


# ---- reduceTo / maxTo over rows folded into the producing kernel ------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16, F16, F64, I32, I16, U8], ids=lambda d: DTYPE_NAMES[d])
@pytest.mark.parametrize("shape", [(1000, 1000), (700, 1001), (4096, 256), (2500, 130)], ids=str)
def test_row_reductions_fused_behind_their_producer(b200, ref, dtype, shape):
    """`y.sum(1)`, `y.max(1)` and `y.sum()` with y's producer still pending: one generated kernel walks y row by row (a CTA
    or a warp per row), stores it and leaves the per-row results; the fills of the destinations travel as kernel scalars.
    Oracle: the CPU device on the same sequence (16-bit floats: reductions on the widened values, rounded once)."""
    rng = np.random.default_rng(700 + dtype + shape[1])
    x, g = values(rng, shape, dtype), values(rng, (shape[1],), dtype)
    if dtype not in FLOATS:
        x, g = x % 7, g % 5
    before = b200.stats()
    tx, tg = TensorValue.from_numpy(x, b200, dtype), TensorValue.from_numpy(g, b200, dtype)
    b200.synchronize()
    y = tx * tg + tx                                     # pending; kept alive, so it is stored as well
    rows_sum, rows_max, total = y.sum(1), y.max(1), y.sum()
    got_y, got_sum, got_max, got_total = y.numpy(), rows_sum.numpy(), rows_max.numpy(), total.numpy()
    after = b200.stats()
    assert after["reductions_fused"] - before["reductions_fused"] == 3, "row reductions were not folded into the producer"
    assert after["fused_kernels"] - before["fused_kernels"] == 1

    rx, rg = TensorValue.from_numpy(x, ref, dtype), TensorValue.from_numpy(g, ref, dtype)
    ry = rx * rg + rx
    want_y = ry.numpy()
    assert_close(got_y, want_y, dtype, "y")
    assert_close(got_max, ry.max(1).numpy(), dtype, "row max")
    if dtype in FLOATS:
        wide_y = ry.to(wide(dtype)) if dtype in (F16, BF16) else ry
        scale = np.maximum(1.0, np.abs(np.asarray(want_y, dtype=np.float64)).sum(axis=1))
        assert_close(got_sum, round_to(wide_y.sum(1).numpy(), dtype), dtype, "row sum", scale=scale)
        exact = np.asarray(want_y, dtype=np.float64).sum()
        bound = {F64: 1e-12, F32: 1e-5, F16: 1e-2, BF16: 1e-2}[dtype]
        assert abs(float(got_total) - exact) <= bound * max(1.0, float(np.abs(np.asarray(want_y, dtype=np.float64)).sum()))
    else:
        assert_close(got_sum, ry.sum(1).numpy(), dtype, "row sum")
        assert_close(got_total, ry.sum().numpy(), dtype, "sum")


def test_fused_row_reduction_accumulates_into_what_the_destination_holds(b200, ref):
    """The device contract is dst += sum(row), dst = max(dst, max(row)): a destination that holds data (not a pending
    fill), and a fill that somebody reads before the reduction, must both be honoured by the fused form."""
    rng = np.random.default_rng(31)
    x = rng.normal(0, 1, (1200, 384)).astype(np.float32)
    start = rng.normal(0, 5, (1200, 1)).astype(np.float32)
    outs = []
    for dev in (b200, ref):
        t = TensorValue.from_numpy(x, dev)
        held_sum, held_max = TensorValue.from_numpy(start, dev), TensorValue.from_numpy(start, dev)
        dev.synchronize()
        before = dev.stats()["reductions_fused"] if dev is b200 else 0
        y = t * 2.0                                       # pending producer
        dev.reduceTo(y.deviceParams(), held_sum.deviceParams())
        dev.maxTo(y.deviceParams(), held_max.deviceParams())
        filled = TensorValue.full(3.0, (1200, 1), dev)
        peek = filled + 1.0                               # reads the fill before the reduction overwrites it
        dev.reduceTo(y.deviceParams(), filled.deviceParams())
        again = filled * 1.0                              # reads the reduction's result
        outs.append((held_sum.numpy(), held_max.numpy(), peek.numpy(), filled.numpy(), again.numpy(), y.numpy()))
        if dev is b200:
            assert dev.stats()["reductions_fused"] - before == 3
    scale = np.abs(x).sum(axis=1, keepdims=True) * 2 + 5
    for k, what in enumerate(("sum into held data", "max into held data", "peek", "sum into a filled destination", "reader after", "y")):
        assert_close(outs[0][k], outs[1][k], F32, what, scale=scale if k in (0, 3, 4) else None)
    assert np.array_equal(outs[0][3], outs[0][4])


def test_row_reduction_fusion_can_be_switched_off(b200):
    """Layouts that do not fit (few rows, short rows, reduced leading dimension) take the stand-alone kernels."""
    rng = np.random.default_rng(5)
    for shape, dim in (((64, 4096), 1), ((4096, 64), 1), ((2048, 512), 0)):
        x = rng.normal(0, 1, shape).astype(np.float32)
        t = TensorValue.from_numpy(x, b200)
        b200.synchronize()
        before = b200.stats()["reductions_fused"]
        got = (t + 1.0).sum(dim).numpy()
        assert b200.stats()["reductions_fused"] == before
        want = (x.astype(np.float64) + 1.0).sum(axis=dim)
        assert np.max(np.abs(got - want)) <= 1e-5 * np.abs(x + 1).sum(axis=dim).max()
