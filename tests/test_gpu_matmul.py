"""matmul parity with the reference's CPU device (Tests/DeviceTests.cpp:1244-1262, 2200-2360, 2806-2875).

f32 results are compared norm-wise (max |diff| / max |C| <= 1e-5): entries of C come arbitrarily close to zero.
For f16/bf16 the oracle is the CPU f32 matmul of the same values, rounded once to the 16-bit type (the CPU device's
own 16-bit accumulator loses everything at large K).
"""
import numpy as np
import pytest

from aix_b200 import BF16, DTYPE_NAMES, F16, F32, F64, I8, I16, I32, I64, U8, TensorValue, from_storage, to_storage

pytestmark = pytest.mark.gpu


def quantize(x, dtype):
    return from_storage(to_storage(x, dtype), dtype)


def normwise(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / max(1e-30, np.max(np.abs(want.astype(np.float64)))))


def check(b200, ref, a, b, dtype, transpose_a=False, transpose_b=False, what=""):
    outs = []
    for dev, dt in ((b200, dtype), (ref, F32 if dtype in (F16, BF16) else dtype)):
        ta = TensorValue.from_numpy(a.T.copy() if transpose_a else a, dev, dt)
        tb = TensorValue.from_numpy(b.T.copy() if transpose_b else b, dev, dt)
        if transpose_a: ta = ta.transpose(0, 1)
        if transpose_b: tb = tb.transpose(0, 1)
        outs.append(ta.matmul(tb).numpy())
    got, want = outs
    if dtype in (I64, I32, I16, I8, U8):
        assert np.array_equal(got, want), what
    else:
        tol = {F64: 1e-12, F32: 1e-5, F16: 1e-2, BF16: 1e-2}[dtype]
        if dtype in (F16, BF16):
            want = quantize(want, dtype)
        assert normwise(got, want) <= tol, f"{what}: norm-wise error {normwise(got, want)}"


@pytest.mark.parametrize("dtype", [F32, F64, BF16, F16, I32, I64, I16, I8, U8], ids=lambda d: DTYPE_NAMES[d])
def test_small_and_odd_shapes(b200, ref, dtype):
    rng = np.random.default_rng(dtype)
    shapes = [(1, 1, 1), (1, 7, 5), (3, 1, 2), (7, 5, 3), (5, 5, 5), (16, 16, 16), (17, 33, 9), (64, 64, 64), (65, 127, 63), (128, 96, 160)]
    for m, k, n in shapes:
        if dtype in (F64, F32, F16, BF16):
            a, b = quantize(rng.normal(0, 1, (m, k)), dtype), quantize(rng.normal(0, 1, (k, n)), dtype)
        else:
            a, b = rng.integers(0, 4, (m, k)), rng.integers(0, 4, (k, n))
        check(b200, ref, a, b, dtype, what=f"{m}x{k}x{n}")


@pytest.mark.parametrize("dtype", [F32, BF16], ids=lambda d: DTYPE_NAMES[d])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_transposed_views_as_operands(b200, ref, dtype, ta, tb):
    """matmul backward feeds stride-swapped views: dA = G . B^T, dB = A^T . G (aixCore.hpp:2192-2207)."""
    rng = np.random.default_rng(17)
    for m, k, n in [(8, 4, 6), (128, 256, 64), (256, 128, 384), (130, 70, 50)]:
        a, b = quantize(rng.normal(0, 0.5, (m, k)), dtype), quantize(rng.normal(0, 0.5, (k, n)), dtype)
        check(b200, ref, a, b, dtype, ta, tb, what=f"{m}x{k}x{n} ta={ta} tb={tb}")


@pytest.mark.parametrize("dtype", [F32, BF16, F16], ids=lambda d: DTYPE_NAMES[d])
def test_medium_sizes_against_float64(b200, dtype):
    """Sizes the CPU device cannot finish in seconds: compare with numpy float64 on the same rounded inputs."""
    rng = np.random.default_rng(23)
    for m, k, n in [(512, 512, 512), (1024, 768, 640), (1000, 1000, 1000), (2048, 1024, 512)]:
        a, b = quantize(rng.normal(0, 0.02, (m, k)), dtype), quantize(rng.normal(0, 0.02, (k, n)), dtype)
        for ta, tb in [(False, False), (False, True), (True, False)]:
            A = TensorValue.from_numpy(a.T.copy() if ta else a, b200, dtype)
            B = TensorValue.from_numpy(b.T.copy() if tb else b, b200, dtype)
            if ta: A = A.transpose(0, 1)
            if tb: B = B.transpose(0, 1)
            got = A.matmul(B).numpy()
            want = a.astype(np.float64) @ b.astype(np.float64)
            tol = 1e-5 if dtype == F32 else 1e-2
            assert normwise(got, want) <= tol, f"{m}x{k}x{n} ta={ta} tb={tb}: {normwise(got, want)}"


def test_f32_operands_of_extreme_and_uneven_magnitude(b200, ref):
    """The f32 product runs on the tensor cores from scaled fp16 terms: the scaling must be invisible - operands far from
    1, operands whose rows differ by many decades, a zero operand - and the result must stay within the f32 bar."""
    rng = np.random.default_rng(23)
    m, k, n = 384, 640, 520
    a = rng.normal(0, 0.5, (m, k)).astype(np.float32)
    b = rng.normal(0, 0.5, (k, n)).astype(np.float32)
    cases = {
        "tiny x huge": (a * np.float32(1e-20), b * np.float32(1e15)),
        "huge x tiny": (a * np.float32(3e30), b * np.float32(1e-35)),
        "rows of different magnitude": ((a * np.exp(rng.uniform(-15, 15, (m, 1)))).astype(np.float32), b),
        "17 decades inside one operand": ((a * np.exp(rng.uniform(-20, 20, a.shape))).astype(np.float32), b),
        "same-sign products": (np.abs(a), np.abs(b)),
    }
    for what, (x, y) in cases.items():
        want = x.astype(np.float64) @ y.astype(np.float64)
        got = TensorValue.from_numpy(x, b200).matmul(TensorValue.from_numpy(y, b200)).numpy()
        assert np.isfinite(got).all(), what
        assert normwise(got, want) <= 1e-5, f"{what}: norm-wise error {normwise(got, want)}"
    zero = TensorValue.from_numpy(np.zeros((m, k), np.float32), b200).matmul(TensorValue.from_numpy(b, b200)).numpy()
    assert not zero.any()


def test_f32_operands_prepared_once_and_never_stale(b200):
    """The tensor-core f32 product keeps the two-term fp16 form of an operand until the operand is written: every
    orientation of one tensor shares it (forward, G.B^T, A^T.G), and any write - a recorded op, an upload, an in-place
    update - must drop it."""
    rng = np.random.default_rng(3)
    m, k, n = 512, 384, 640
    a, b = rng.normal(0, 0.5, (m, k)).astype(np.float32), rng.normal(0, 0.5, (k, n)).astype(np.float32)
    A, B = TensorValue.from_numpy(a, b200), TensorValue.from_numpy(b, b200)
    G = TensorValue.from_numpy(rng.normal(0, 0.5, (m, n)).astype(np.float32), b200)
    g = G.numpy()
    s0 = b200.stats()
    c = A.matmul(B).numpy()
    da = G.matmul(B.transpose(0, 1)).numpy()            # B again, now K-major instead of MN-major
    db = A.transpose(0, 1).matmul(G).numpy()            # A and G again, both MN-major
    s1 = b200.stats()
    assert s1["prepared_operand_builds"] - s0["prepared_operand_builds"] == 3, "A, B and G are prepared once each"
    assert s1["prepared_operand_hits"] - s0["prepared_operand_hits"] == 3
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), g.astype(np.float64)
    assert normwise(c, a64 @ b64) <= 1e-5 and normwise(da, g64 @ b64.T) <= 1e-5 and normwise(db, a64.T @ g64) <= 1e-5
    # a recorded in-place update of B, an upload into A, a full overwrite of G: every later product sees the new values
    B *= 2.0
    a2 = rng.normal(0, 0.5, (m, k)).astype(np.float32)
    b200.copy(a2.ctypes.data, F32, A.storage.data, F32, a2.size)
    assert normwise(A.matmul(B).numpy(), a2.astype(np.float64) @ (2.0 * b64)) <= 1e-5
    b200.fill(1.0, F32, G.deviceParams())
    assert normwise(A.transpose(0, 1).matmul(G).numpy(), a2.astype(np.float64).T @ np.ones((m, n))) <= 1e-5
    # a view of part of a tensor, and a write into another part of the same storage
    big = TensorValue.from_numpy(rng.normal(0, 0.5, (2 * m, k)).astype(np.float32), b200)
    upper = TensorValue(big.storage, (m, k), (k, 1), 0, F32, b200)
    lower = TensorValue(big.storage, (m, k), (k, 1), m * k, F32, b200)
    want = big.numpy().astype(np.float64)
    first = upper.matmul(B).numpy()
    lower *= 0.0                                         # does not touch `upper`
    again = upper.matmul(B).numpy()
    assert np.array_equal(first, again) and normwise(first, want[:m] @ (2.0 * b64)) <= 1e-5
    upper += 1.0
    assert normwise(upper.matmul(B).numpy(), (want[:m] + 1.0) @ (2.0 * b64)) <= 1e-5
    # freed and reused storage: a new tensor in the old block is a new operand
    for scale in (1.0, 3.0):
        t = TensorValue.from_numpy(a * np.float32(scale), b200)
        assert normwise(t.matmul(B).numpy(), (a64 * scale) @ (2.0 * b64)) <= 1e-5
        del t
