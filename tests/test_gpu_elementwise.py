"""Device-vs-CPU parity of the recorded elementwise ops, through the C ABI.

Modelled on the reference's device parity tests (Targets/AIXTests/DeviceTests.cpp:198-560): the same op is run on the
device under test and on the reference's CPU device over a ladder of sizes around the vector widths and for all
nine element types; integers must match exactly, floats within the stated tolerance.
"""
import numpy as np
import pytest

from aix_b200 import (BF16, DTYPE_NAMES, F16, F32, F64, I8, I16, I32, I64, U8, TensorValue, scalar_like)
from conftest import assert_close

pytestmark = pytest.mark.gpu

SIZES = [1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 129, 255, 257, 511, 1023, 1025, 2047, 2049, 100003]
ALL_DTYPES = [F64, F32, F16, BF16, I64, I32, I16, I8, U8]
FLOATS = [F64, F32, F16, BF16]


def make_input(rng, n, dtype, positive=False, small=False):
    if dtype in FLOATS:
        lo = 0.1 if positive else -2.0
        return rng.uniform(lo, 2.0, n)
    if dtype == U8:
        return rng.integers(1 if positive else 0, 12 if small else 200, n)
    lo = 1 if positive else (-6 if small else -90)
    v = rng.integers(lo, 7 if small else 90, n)
    return v


def run_binary(dev, op, x, y, dtype):
    a = TensorValue.from_numpy(x, dev, dtype)
    b = TensorValue.from_numpy(y, dev, dtype)
    ops = {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "div": lambda: a / b, "pow": lambda: a.pow(b)}
    return ops[op]().numpy()


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=lambda d: DTYPE_NAMES[d])
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "pow"])
def test_binary_ops_match_cpu_device(b200, ref, op, dtype):
    rng = np.random.default_rng(1234 + dtype)
    for n in SIZES:
        x = make_input(rng, n, dtype, positive=(op == "pow"), small=(op in ("mul", "pow")))
        y = make_input(rng, n, dtype, positive=(op in ("div", "pow")), small=(op in ("mul", "pow")))
        if op == "pow" and dtype not in FLOATS:
            y = np.minimum(y, 3)
        got = run_binary(b200, op, x, y, dtype)
        want = run_binary(ref, op, x, y, dtype)
        assert_close(got, want, dtype, f"{op} {DTYPE_NAMES[dtype]} n={n}")


def run_unary(dev, op, x, dtype):
    a = TensorValue.from_numpy(x, dev, dtype)
    r = -a if op == "neg" else getattr(a, op)()
    return r.numpy(), r.dtype


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=lambda d: DTYPE_NAMES[d])
@pytest.mark.parametrize("op", ["neg", "sqrt", "sin", "cos", "tanh", "log", "exp"])
def test_unary_ops_match_cpu_device(b200, ref, op, dtype):
    rng = np.random.default_rng(99 + dtype)
    for n in SIZES:
        x = make_input(rng, n, dtype, positive=(op in ("sqrt", "log")), small=(op == "exp"))
        got, gdt = run_unary(b200, op, x, dtype)
        want, wdt = run_unary(ref, op, x, dtype)
        assert gdt == wdt
        assert_close(got, want, gdt, f"{op} {DTYPE_NAMES[dtype]} n={n}")


def test_unary_device_calls_on_integer_tensors(b200, ref):
    """Device::sqrt/exp/sin... called directly on integer tensors: wide-float math, saturating conversion back
    (aixDeviceCPU.cpp:155-242)."""
    rng = np.random.default_rng(5)
    for dtype in (I64, I32, I16, I8, U8):
        x = make_input(rng, 777, dtype, positive=True, small=True)
        for op in ("sqrt", "sin", "cos", "tanh", "log", "exp"):
            outs = []
            for dev in (b200, ref):
                a = TensorValue.from_numpy(x, dev, dtype)
                r = TensorValue.empty(a.shape, dev, dtype)
                getattr(dev, op)(a.deviceParams(), r.deviceParams())
                outs.append(r.numpy())
            assert_close(outs[0], outs[1], dtype, f"{op} on {DTYPE_NAMES[dtype]}")


def chain(dev, a, b, c, dtype=F32):
    """Config-0 expression with Tensor-level scalars (one-element fills broadcast with zero strides)."""
    ta, tb, tc = (TensorValue.from_numpy(v, dev, dtype) for v in (a, b, c))
    one = lambda t: scalar_like(1.0, t)
    z = (ta * tb + tc) * (one(ta) / (one(ta) + (-ta).exp())) - tb.tanh() / (one(tc) + (-tc).exp())
    return z, z.sum()


def test_config0_chain_matches_reference_front_end(b200, ref):
    """z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c)), s = z.sum() on [1024,1024] f32, U(-1,1), seed 0,
    against the reference's own aix::Tensor front end on its CPU device."""
    rng = np.random.default_rng(0)
    a, b, c = (rng.uniform(-1, 1, (1024, 1024)).astype(np.float32) for _ in range(3))
    before = b200.stats()
    z, s = chain(b200, a, b, c)
    got_z, got_s = z.numpy(), float(s.item())
    after = b200.stats()
    want_z, want_s, _ = ref.chain_f32(a, b, c)
    assert_close(got_z, want_z, F32, "chain z")
    # The reference's f32 sum is a sequential accumulation and is itself ~1e-5 away from the exact sum:
    # compare against the float64 sum of the reference's z, and bound the distance to its f32 sum by the data.
    exact = float(want_z.astype(np.float64).sum())
    assert abs(got_s - exact) <= 1e-5 * max(1.0, abs(exact))
    assert abs(got_s - want_s) <= 1e-5 * float(np.abs(want_z).astype(np.float64).sum())
    # one generated kernel for the 13-op expression, nothing but z written
    assert after["fused_kernels"] - before["fused_kernels"] == 1
    assert after["fused_ops"] - before["fused_ops"] >= 13
    assert after["fills_absorbed"] - before["fills_absorbed"] == 3


@pytest.mark.parametrize("dtype", [F32, BF16, F16, F64], ids=lambda d: DTYPE_NAMES[d])
def test_chain_all_float_types_match_cpu_device(b200, ref, dtype):
    rng = np.random.default_rng(7)
    a, b, c = (rng.uniform(-1, 1, (257, 131)) for _ in range(3))
    got, _ = chain(b200, a, b, c, dtype)
    want, _ = chain(ref, a, b, c, dtype)
    assert_close(got.numpy(), want.numpy(), dtype, "chain")


def test_broadcast_views(b200, ref):
    """Row, column, scalar and general strided operands (Tests/DeviceTests.cpp:1682-1760)."""
    rng = np.random.default_rng(3)
    for dtype in (F32, BF16, I32):
        for (r, c) in [(5, 7), (64, 128), (33, 1000), (128, 36)]:
            x = make_input(rng, r * c, dtype).reshape(r, c)
            row = make_input(rng, c, dtype)
            col = make_input(rng, r, dtype).reshape(r, 1)
            outs = []
            for dev in (b200, ref):
                tx = TensorValue.from_numpy(x, dev, dtype)
                trow = TensorValue.from_numpy(row, dev, dtype)
                tcol = TensorValue.from_numpy(col, dev, dtype)
                y = tx * trow + tcol                      # (0,1) and (1,0) broadcast strides
                y = y - tx.transpose(0, 1).contiguous().transpose(0, 1)   # general strided operand
                y = y + scalar_like(3.0, y)
                outs.append(y.numpy())
            assert_close(outs[0], outs[1], dtype, f"broadcast {DTYPE_NAMES[dtype]} {r}x{c}")


def test_in_place_sequence_keeps_program_order(b200, ref):
    """m *= 0.9; m += 0.1*g; out = m / 0.5 (Tests/DeviceTests.cpp:1882-1910)."""
    rng = np.random.default_rng(11)
    g0, m0 = rng.uniform(-1, 1, 4099).astype(np.float32), rng.uniform(-1, 1, 4099).astype(np.float32)
    outs = []
    for dev in (b200, ref):
        g, m = TensorValue.from_numpy(g0, dev), TensorValue.from_numpy(m0, dev)
        for _ in range(3):
            m *= 0.9
            m += 0.1 * g
        out = m / 0.5
        outs.append((out.numpy(), m.numpy()))
    assert_close(outs[0][0], outs[1][0], F32, "out")
    assert_close(outs[0][1], outs[1][1], F32, "m")


def test_kernel_cache_is_shared_across_scalar_values(b200):
    """x*2+1 and x*3+5 use one kernel: scalars are runtime arguments (Tests/DeviceTests.cpp:1774-1807)."""
    x = TensorValue.from_numpy(np.array([[1, 2], [3, 4]], dtype=np.float32), b200)
    y1 = (x * 2.0 + 1.0).numpy()
    s1 = b200.stats()
    y2 = (x * 3.0 + 5.0).numpy()
    s2 = b200.stats()
    assert y1.reshape(-1).tolist() == [3, 5, 7, 9]
    assert y2.reshape(-1).tolist() == [8, 11, 14, 17]
    assert s2["kernel_cache_misses"] == s1["kernel_cache_misses"]
    assert s2["kernel_cache_hits"] > s1["kernel_cache_hits"]


def test_fill_conversions_saturate(b200, ref):
    """fill converts float scalars to integer tensors with saturation and NaN -> 0 (Tests/DeviceTests.cpp:1282-1332)."""
    for dtype in (I64, I32, I16, I8, U8, F16, BF16, F32, F64):
        for value in (3.7, -3.7, 1e10, -1e10, 300.0, -300.0, float("nan"), 0.0):
            outs = []
            for dev in (b200, ref):
                t = TensorValue.full(value, (37,), dev, dtype)
                outs.append(t.raw())
            if np.isnan(value) and dtype in FLOATS:
                continue
            assert np.array_equal(outs[0], outs[1]), f"fill {value} -> {DTYPE_NAMES[dtype]}"


def test_dtype_conversion_copy(b200, ref):
    rng = np.random.default_rng(2)
    x = rng.uniform(-300, 300, 1001)
    for src in ALL_DTYPES:
        for dst in ALL_DTYPES:
            outs = []
            for dev in (b200, ref):
                t = TensorValue.from_numpy(np.clip(x, 0, 200) if src == U8 else x, dev, src)
                outs.append(t.to(dst).raw())
            assert np.array_equal(outs[0], outs[1]), f"copy {DTYPE_NAMES[src]} -> {DTYPE_NAMES[dst]}"


def test_long_chain_without_synchronize(b200, ref):
    """1024 in-place adds on one tensor, one synchronize at the end (Tests/DeviceTests.cpp:3478-3500)."""
    x = TensorValue.full(1.0, (1 << 16,), b200)
    y = TensorValue.full(1.0, (1 << 16,), b200)
    for _ in range(1024):
        x += y
    assert np.all(x.numpy() == 1025.0)
