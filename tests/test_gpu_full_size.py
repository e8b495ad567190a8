"""The benchmark configurations at their FULL sizes on the B200 device, held against the reference.

The reference's CPU device cannot finish these sizes in seconds (its matmul runs near 0.14 GFLOP/s), so each case is
checked through pieces the CPU device can do plus size-independent properties:
  * rows of an elementwise result are independent, so sampled row blocks go through the CPU device op by op;
  * reductions of the GPU's own (downloaded) elementwise result go through the CPU device / float64;
  * matmul and the MLP step are held norm-wise against float64 numpy on the whole result, and against the CPU device on a
    slab of rows.
Tolerances: f32 1e-5 (norm-wise for matmul, relative to sum |x| for sums), bf16 1e-2, exact where the value is exact.
"""
import numpy as np
import pytest

from aix_b200 import BF16, F32, TensorValue, from_storage, to_storage
from aix_b200.frontend import Linear, MSELoss, Sequential, Tanh, Tensor
from aix_b200.mlp import DEFAULT_DIMS, MlpTrainer, synthetic_batch, xavier_parameters
from conftest import assert_close

pytestmark = pytest.mark.gpu


def quantize(x, dtype):
    return from_storage(to_storage(x, dtype), dtype)


def normwise(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - want)) / max(1e-300, np.max(np.abs(want))))


def relu(v):
    return (v + (v * v).sqrt()) * 0.5


# ---- configuration 1: broadcast + reductions, bf16 storage, 8192 x 8192 ----------------------------------------------------
def test_config1_full_size_bf16(b200, ref):
    rows = cols = 8192
    rng = np.random.default_rng(0)
    x = quantize(rng.normal(0, 1, (rows, cols)).astype(np.float32), BF16)
    g = quantize(rng.uniform(0.5, 1.5, cols).astype(np.float32), BF16)
    bias = quantize(rng.normal(0, 0.1, cols).astype(np.float32), BF16)
    tx, tg, tb = (TensorValue.from_numpy(v, b200, BF16) for v in (x, g, bias))
    y = relu(tx * tg + tb)
    row_sum, row_max, mean = y.sum(1), y.max(1), y.mean()
    got_y, got_sum, got_max, got_mean = y.numpy(), row_sum.numpy(), row_max.numpy(), float(mean.numpy())

    # y: the same op sequence on the CPU device for sampled row blocks (every row is independent of the others)
    picked = np.concatenate([np.arange(0, 64), rng.choice(np.arange(64, rows - 64), 128, replace=False), np.arange(rows - 64, rows)])
    rx, rg, rb = (TensorValue.from_numpy(v, ref, BF16) for v in (x[picked], g, bias))
    want_rows = relu(rx * rg + rb).numpy()
    assert_close(got_y[picked], want_rows, BF16, "y on sampled rows")
    assert (got_y >= 0).all()

    # row maxima are exact; row sums: the CPU device on the f32-widened rows of the GPU's own y, rounded once to bf16
    assert np.array_equal(got_max, got_y.max(axis=1)), "row max"
    wide = TensorValue.from_numpy(got_y, ref, F32)
    want_sum = quantize(wide.sum(1).numpy(), BF16)
    assert_close(got_sum, want_sum, BF16, "row sum", scale=np.maximum(1.0, np.abs(want_sum)))
    exact_rows = got_y.astype(np.float64).sum(axis=1)
    assert np.max(np.abs(got_sum - exact_rows) / exact_rows) <= 2.0 ** -8, "row sums: within half a bf16 ulp of the float64 sums"

    # global mean = sum() / size with both operands in bf16 (aixCore.hpp:2498-2501); size = 2^26 is exact in bf16
    total = float(quantize(np.array([got_y.astype(np.float64).sum()]), BF16)[0])
    want_mean = float(quantize(np.array([total / float(rows * cols)]), BF16)[0])
    assert abs(got_mean - want_mean) <= 1e-2 * abs(want_mean), (got_mean, want_mean)


# ---- configuration 2: 4096^3 matmul with autograd backward from a seed of ones --------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(F32, 1e-5), (BF16, 1e-2)], ids=["f32", "bf16"])
def test_config2_matmul_forward_and_autograd_backward_4096(b200, ref, dtype, tol):
    n = 4096
    rng = np.random.default_rng(0)
    a = quantize(rng.normal(0, 0.02, (n, n)).astype(np.float32), dtype)
    b = quantize(rng.normal(0, 0.02, (n, n)).astype(np.float32), dtype)
    A = Tensor(TensorValue.from_numpy(a, b200, dtype), requireGrad=True)
    B = Tensor(TensorValue.from_numpy(b, b200, dtype), requireGrad=True)
    C = A.matmul(B)
    C.backward()                                        # seed of ones: dA = 1 . B^T, dB = A^T . 1 (aixCore.hpp:2192-2207)
    got_c, got_da, got_db = C.value.numpy(), A.grad().numpy(), B.grad().numpy()

    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    want_c = a64 @ b64
    want_da = np.broadcast_to(b64.sum(axis=1)[None, :], (n, n))      # dA[i, j] = sum_n B[j, n]
    want_db = np.broadcast_to(a64.sum(axis=0)[:, None], (n, n))      # dB[k, j] = sum_m A[m, k]
    for what, got, want in (("C", got_c, want_c), ("dA", got_da, want_da), ("dB", got_db, want_db)):
        assert np.isfinite(got).all(), what
        assert normwise(got, want) <= tol, f"{what}: norm-wise error {normwise(got, want):.3g}"

    # a slab of rows through the reference's CPU device (f32 accumulation; for bf16 the operands are widened first,
    # the CPU device's own bf16 accumulator loses everything at K = 4096)
    slab = rng.choice(n, 8, replace=False)
    ra, rb = TensorValue.from_numpy(a[slab], ref, F32), TensorValue.from_numpy(b, ref, F32)
    want_slab = ra.matmul(rb).numpy()
    if dtype == BF16:
        want_slab = quantize(want_slab, BF16)
    assert normwise(got_c[slab], want_slab) <= tol, f"slab vs CPU device: {normwise(got_c[slab], want_slab):.3g}"


# ---- configuration 3: one full-width MLP training step ---------------------------------------------------------------------
def test_config3_full_width_step_against_float64(b200):
    dims, batch = DEFAULT_DIMS, 4096
    weights, biases = xavier_parameters(dims, seed=0)
    x, y = synthetic_batch(dims, batch)
    layers = []
    for i, (w, bvec) in enumerate(zip(weights, biases)):
        layers.append(Linear(w, bvec + np.float32(0.01) * (i + 1), b200))       # non-zero biases so the bias path is exercised
        if i + 1 < len(weights):
            layers.append(Tanh())
    tx, ty = Tensor(TensorValue.from_numpy(x, b200)), Tensor(TensorValue.from_numpy(y, b200))
    activations, h = [], tx
    for m in layers:
        h = m.forward(h)
        if isinstance(m, Tanh):
            activations.append(h)
    loss = MSELoss()(h, ty)
    for m in layers:
        for p in m.parameters():
            p.zeroGrad()
    loss.backward()

    # float64 forward and backward on the host
    w64 = [w.astype(np.float64) for w in weights]
    b64 = [(bv + np.float32(0.01) * (i + 1)).astype(np.float64) for i, bv in enumerate(biases)]
    hs, cur = [x.astype(np.float64)], x.astype(np.float64)
    for i in range(4):
        cur = cur @ w64[i] + b64[i]
        if i < 3:
            cur = np.tanh(cur)
        hs.append(cur)
    diff = hs[4] - y.astype(np.float64)
    want_loss = float(np.mean(diff * diff))
    got_loss = float(loss.value.item())
    assert abs(got_loss - want_loss) <= 1e-5 * want_loss, (got_loss, want_loss)

    rows = np.random.default_rng(1).choice(batch, 64, replace=False)
    for i, act in enumerate(activations):
        got = act.value.numpy()[rows]
        # tanh outputs lie in [-1, 1]: absolute = norm-wise. The first layer is one matmul away from the inputs (1e-5); the
        # later ones inherit the earlier layers' rounding through another 4096-term contraction each (2e-5).
        assert np.max(np.abs(got - hs[i + 1][rows])) <= (1e-5 if i == 0 else 2e-5), f"activation {i + 1}"
    assert normwise(h.value.numpy()[rows], hs[4][rows]) <= 2e-5, "prediction"

    grad = 2.0 * diff / diff.size
    linear = [m for m in layers if isinstance(m, Linear)]
    for i in (3, 2, 1, 0):
        want_dw, want_db = hs[i].T @ grad, grad.sum(axis=0, keepdims=True)
        got_dw, got_db = linear[i].w.grad().numpy(), linear[i].b.grad().numpy()
        assert normwise(got_dw, want_dw) <= 2e-5, f"dW{i + 1}: {normwise(got_dw, want_dw):.3g}"
        assert normwise(got_db, want_db) <= 2e-5, f"db{i + 1}: {normwise(got_db, want_db):.3g}"
        if i > 0:
            grad = (grad @ w64[i].T) * (1.0 - hs[i] * hs[i])


def test_config3_hundred_steps_follow_the_reference_front_end(b200, ref):
    """Configuration 3 runs 100 steps: the loss curve of a reduced-width model against the reference's own front end on
    its CPU device, over all 100 steps (the full width would take the CPU device hours)."""
    dims, batch, steps = (32, 128, 128, 128, 32), 64, 100
    weights, biases = xavier_parameters(dims, seed=0)
    x, y = synthetic_batch(dims, batch)
    trainer = MlpTrainer(b200, dims, batch, weights=[w.copy() for w in weights], biases=[b.copy() for b in biases])
    got = np.array([float(trainer.step().value.item()) for _ in range(steps)])
    ref_w, ref_b = [w.copy() for w in weights], [b.copy() for b in biases]
    want, _ = ref.mlp_train_f32(list(dims), ref_w, ref_b, x, y, steps, lr=1e-3)
    assert np.allclose(got[:20], want[:20], rtol=5e-5), (got[:20], want[:20])
    assert np.allclose(got, want, rtol=2e-3), np.max(np.abs(got - want) / want)
    assert got[-1] < 0.9 * got[0]
    params = trainer.parameters_numpy()
    for i in range(4):
        for g, w in ((params[2 * i], ref_w[i]), (params[2 * i + 1], ref_b[i])):
            assert np.mean(np.abs(g - w)) <= 2e-5


# ---- strict math: a second device handle with contraction and approximate routines switched off ---------------------------
@pytest.fixture(scope="module")
def strict():
    from aix_b200 import DeviceB200
    dev = DeviceB200(0, strict_math=1)
    yield dev
    dev.synchronize()
    dev.close()


def test_strict_math_elementwise_ladder_and_chain(strict, ref):
    from aix_b200 import scalar_like
    rng = np.random.default_rng(77)
    unary = {"neg": lambda t: -t, "sqrt": lambda t: t.sqrt(), "sin": lambda t: t.sin(), "cos": lambda t: t.cos(), "tanh": lambda t: t.tanh(),
             "log": lambda t: t.log(), "exp": lambda t: t.exp()}
    binary = {"add": lambda p, q: p + q, "sub": lambda p, q: p - q, "mul": lambda p, q: p * q, "div": lambda p, q: p / q, "pow": lambda p, q: p.pow(q)}
    for dtype in (F32, BF16):
        for n in (1, 3, 4, 5, 17, 63, 129, 1025, 2049, 100003):
            x = rng.uniform(0.1, 2.0, n)
            y = rng.uniform(0.1, 2.0, n)
            for name, fn in unary.items():
                got = fn(TensorValue.from_numpy(x, strict, dtype)).numpy()
                want = fn(TensorValue.from_numpy(x, ref, dtype)).numpy()
                assert_close(got, want, dtype, f"strict {name} n={n}")
            for name, fn in binary.items():
                got = fn(TensorValue.from_numpy(x, strict, dtype), TensorValue.from_numpy(y, strict, dtype)).numpy()
                want = fn(TensorValue.from_numpy(x, ref, dtype), TensorValue.from_numpy(y, ref, dtype)).numpy()
                assert_close(got, want, dtype, f"strict {name} n={n}")
    # the config-0 expression at its own size, against the reference front end on its CPU device
    a, b, c = (rng.uniform(-1, 1, (1024, 1024)).astype(np.float32) for _ in range(3))
    ta, tb, tc = (TensorValue.from_numpy(v, strict) for v in (a, b, c))
    one = lambda t: scalar_like(1.0, t)
    z = (ta * tb + tc) * (one(ta) / (one(ta) + (-ta).exp())) - tb.tanh() / (one(tc) + (-tc).exp())
    s = z.sum()
    want_z, _want_s, _ = ref.chain_f32(a, b, c)
    got_z = z.numpy()
    assert np.max(np.abs(got_z - want_z) / np.maximum(1.0, np.abs(want_z))) <= 5e-7, "strict mode: a few ulps from the CPU device at most"
    exact = float(want_z.astype(np.float64).sum())
    assert abs(float(s.item()) - exact) <= 1e-5 * float(np.abs(want_z).astype(np.float64).sum())
    assert strict.stats()["fused_kernels"] >= 1


# ---- host memory as an operand of the immediate ops ------------------------------------------------------------------------
def test_host_operands_of_matmul_reduce_and_binary_ops(b200, ref):
    """The reference's device tests hand CPU-resident tensors straight to the device under test
    (Tests/DeviceTests.cpp:209-216): operands in plain host memory are staged, results live on the device. The staging
    blocks must stay intact until the consuming kernels are enqueued, also when the op needs temporaries of the same
    size (f32 matmul with K a multiple of 128)."""
    from aix_b200 import DeviceTensorParams
    rng = np.random.default_rng(5)

    def host(v):
        v = np.ascontiguousarray(v, dtype=np.float32)
        shape = v.shape
        strides = tuple(int(s // 4) for s in v.strides)
        return v, DeviceTensorParams(v.ctypes.data, F32, 0, shape, v.size, strides)

    for m, k, n in [(256, 384, 256), (128, 128, 128), (512, 256, 384)]:
        a, pa = host(rng.normal(0, 0.5, (m, k)))
        b, pb = host(rng.normal(0, 0.5, (k, n)))
        out = TensorValue.empty((m, n), b200)
        b200.matmul(pa, pb, out.deviceParams())
        want = a.astype(np.float64) @ b.astype(np.float64)
        assert normwise(out.numpy(), want) <= 1e-5, f"matmul {m}x{k}x{n} from host operands"
        # mixed: one operand on the device
        out2 = TensorValue.empty((m, n), b200)
        on_device = TensorValue.from_numpy(a, b200)                    # kept alive across the call
        b200.matmul(on_device.deviceParams(), pb, out2.deviceParams())
        assert normwise(out2.numpy(), want) <= 1e-5

    x, px = host(rng.normal(0, 1, (300, 500)))
    y, py = host(rng.normal(0, 1, (300, 500)))
    for name in ("add", "sub", "mul", "div"):
        out = TensorValue.empty(x.shape, b200)
        getattr(b200, name)(px, py, out.deviceParams())
        want = TensorValue.empty(x.shape, ref)
        getattr(ref, name)(px, py, want.deviceParams())
        assert_close(out.numpy(), want.numpy(), F32, f"{name} from host operands")
    col = TensorValue.full(0.0, (1, 500), b200)
    b200.reduceTo(px, col.deviceParams())
    want = TensorValue.full(0.0, (1, 500), ref)
    ref.reduceTo(px, want.deviceParams())
    assert_close(col.numpy(), want.numpy(), F32, "reduceTo from a host operand", scale=np.abs(x).sum(axis=0, keepdims=True))
    total = TensorValue.empty((), b200)
    b200.sum(px, total.deviceParams())
    assert abs(float(total.numpy()) - float(x.astype(np.float64).sum())) <= 1e-5 * float(np.abs(x).sum())


# ---- indices outside the indexed dimension are skipped and reported, never followed ---------------------------------------
def test_index_ops_skip_and_report_out_of_range_indices(b200):
    from aix_b200 import I32
    x = np.arange(40, dtype=np.float32).reshape(8, 5)
    for bad in ([1, 9, 3], [-1, 2, 4]):
        t = TensorValue.from_numpy(x, b200)
        idx = TensorValue.from_numpy(np.array(bad), b200, I32)
        sel = TensorValue.full(-7.0, (3, 5), b200)
        b200.synchronize()
        b200.indexSelect(t.deviceParams(), sel.deviceParams(), idx.deviceParams(), 0)
        with pytest.raises(ValueError, match="outside the indexed dimension"):
            b200.synchronize()
        got = sel.numpy()                                   # the device is usable again; valid rows landed, the bad one was skipped
        assert np.array_equal(got[0], x[bad[0]]) if bad[0] >= 0 else np.all(got[0] == -7.0)
        assert np.all(got[[i for i, v in enumerate(bad) if v < 0 or v >= 8]] == -7.0)
        assert np.array_equal(got[2], x[bad[2]])
        acc = TensorValue.from_numpy(np.zeros((8, 5), np.float32), b200)
        src = TensorValue.from_numpy(np.ones((3, 5), np.float32), b200)
        b200.synchronize()
        b200.indexAdd(src.deviceParams(), acc.deviceParams(), idx.deviceParams(), 0)
        with pytest.raises(ValueError, match="outside the indexed dimension"):
            b200.synchronize()
        want = np.zeros((8, 5), np.float32)
        for v in bad:
            if 0 <= v < 8:
                want[v] += 1.0
        assert np.array_equal(acc.numpy(), want)
    # a strided index tensor is read through its strides
    every_other = TensorValue.from_numpy(np.array([0, 99, 2, 99, 4, 99]), b200, I32)
    view = TensorValue(every_other.storage, (3,), (2,), 0, I32, b200)
    sel = TensorValue.empty((3, 5), b200)
    source = TensorValue.from_numpy(x, b200)
    b200.indexSelect(source.deviceParams(), sel.deviceParams(), view.deviceParams(), 0)
    assert np.array_equal(sel.numpy(), x[[0, 2, 4]])


def test_index_select_by_whole_runs_skips_out_of_range_indices_too(b200):
    """Slices long enough to be copied as contiguous runs take another kernel: same rule, same report."""
    from aix_b200 import I32
    x = np.arange(100 * 64, dtype=np.float32).reshape(100, 64)
    bad = np.arange(80) % 100
    bad[7], bad[50] = 100, -3
    t = TensorValue.from_numpy(x, b200)
    idx = TensorValue.from_numpy(bad, b200, I32)
    sel = TensorValue.full(-7.0, (80, 64), b200)
    b200.synchronize()
    b200.indexSelect(t.deviceParams(), sel.deviceParams(), idx.deviceParams(), 0)
    with pytest.raises(ValueError, match="outside the indexed dimension"):
        b200.synchronize()
    got = sel.numpy()
    for row, v in enumerate(bad):
        assert (np.array_equal(got[row], x[v]) if 0 <= v < 100 else np.all(got[row] == -7.0)), row
