"""Parity of the remaining aix::Device virtuals (argmax family, transpose, sliceSet, tril/triu, indexSelect, indexAdd)
with the reference's CPU device: same device calls, same descriptors, results compared element for element
(Tests/DeviceTests.cpp:729-1240, 1990-2360)."""
import numpy as np
import pytest

from aix_b200 import BF16, DTYPE_NAMES, F16, F32, F64, I8, I16, I32, I64, U8, TensorValue
from conftest import assert_close

pytestmark = pytest.mark.gpu
DTYPES = [F32, F64, BF16, F16, I32, I64, I16, I8, U8]      # all nine, as Tests/DeviceTests.cpp:30-33


def values(rng, shape, dtype):
    if dtype in (F32, F64, BF16, F16):
        return np.round(rng.normal(0, 4, shape), 2)
    return rng.integers(0 if dtype == U8 else -50, 50, shape)


def both(b200, ref, fn):
    return fn(b200), fn(ref)


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_argmax_family(b200, ref, dtype):
    rng = np.random.default_rng(300 + dtype)
    for shape in [(7,), (5, 9), (3, 4, 6), (130, 33)]:
        x = values(rng, shape, dtype)

        def run(dev):
            t = TensorValue.from_numpy(x, dev, dtype)
            out = []
            for view in (t, t.transpose(0, len(shape) - 1)):
                r = TensorValue.empty((), dev, I32)
                dev.argmax(view.deviceParams(), r.deviceParams())
                oh = TensorValue.empty(view.shape, dev, I32)
                dev.argmaxIndices(view.deviceParams(), oh.deviceParams())
                out += [r.numpy(), oh.numpy()]
            for dim in range(len(shape)):
                red = list(shape)
                red[dim] = 1
                r = TensorValue.empty(red, dev, I32)
                dev.argmaxTo(t.deviceParams(), r.deviceParams(), dim)
                oh = TensorValue.full(0, shape, dev, I32)
                dev.argmaxIndicesTo(t.deviceParams(), oh.deviceParams(), dim)
                out += [r.numpy(), oh.numpy()]
            return out
        got, want = both(b200, ref, run)
        for i, (g, w) in enumerate(zip(got, want)):
            assert np.array_equal(g, w), f"{DTYPE_NAMES[dtype]} {shape} output {i}"


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_transpose_materialised(b200, ref, dtype):
    rng = np.random.default_rng(400 + dtype)
    for shape, (d0, d1) in [((4, 7), (0, 1)), ((3, 5, 6), (0, 2)), ((3, 5, 6), (1, 2)), ((2, 3, 4, 5), (1, 3)), ((65, 130), (0, 1))]:
        x = values(rng, shape, dtype)

        def run(dev):
            t = TensorValue.from_numpy(x, dev, dtype)
            new_shape = list(shape)
            new_shape[d0], new_shape[d1] = new_shape[d1], new_shape[d0]
            r = TensorValue.empty(new_shape, dev, dtype)
            dev.transpose(t.deviceParams(), r.deviceParams(), d0, d1)
            return r.raw()
        got, want = both(b200, ref, run)
        assert np.array_equal(got, want), f"{DTYPE_NAMES[dtype]} {shape} {d0},{d1}"


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_slice_set_tril_triu(b200, ref, dtype):
    rng = np.random.default_rng(500 + dtype)
    for shape, dim, start, end, step in [((8,), 0, 2, 7, 1), ((6, 9), 1, 1, 9, 3), ((6, 9), 0, 0, 6, 2), ((3, 4, 10), 2, 3, 10, 2), ((40, 70), 0, 5, 37, 4)]:
        extent = (end - start + step - 1) // step
        src_shape = list(shape)
        src_shape[dim] = extent
        x, base = values(rng, src_shape, dtype), values(rng, shape, dtype)

        def run(dev):
            s = TensorValue.from_numpy(x, dev, dtype)
            d = TensorValue.from_numpy(base, dev, dtype)
            dev.sliceSet(s.deviceParams(), d.deviceParams(), dim, start, end, step)
            return d.raw()
        got, want = both(b200, ref, run)
        assert np.array_equal(got, want), f"sliceSet {DTYPE_NAMES[dtype]} {shape}"
    for shape in [(5, 5), (4, 7), (3, 6, 4), (33, 65)]:
        x = values(rng, shape, dtype)
        for diagonal in (-2, 0, 1, 3):
            def run(dev):
                t = TensorValue.from_numpy(x, dev, dtype)
                lo, up = TensorValue.empty(shape, dev, dtype), TensorValue.empty(shape, dev, dtype)
                dev.tril(t.deviceParams(), lo.deviceParams(), diagonal)
                dev.triu(t.deviceParams(), up.deviceParams(), diagonal)
                return lo.raw(), up.raw()
            got, want = both(b200, ref, run)
            assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]), f"tril/triu {DTYPE_NAMES[dtype]} {shape} {diagonal}"


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_index_select_and_index_add(b200, ref, dtype):
    rng = np.random.default_rng(600 + dtype)
    for shape, dim, idx in [((9,), 0, [3, 0, 8, 3]), ((5, 6), 0, [4, 4, 1]), ((5, 6), 1, [0, 5, 2, 2, 3]), ((3, 4, 5), 1, [3, 1]), ((40, 33), 1, list(range(0, 33, 3)))]:
        x = values(rng, shape, dtype)
        src_shape = list(shape)
        src_shape[dim] = len(idx)
        add = values(rng, src_shape, dtype)

        def run(dev):
            t = TensorValue.from_numpy(x, dev, dtype)
            indices = TensorValue.from_numpy(np.array(idx), dev, I32)
            sel = TensorValue.empty(src_shape, dev, dtype)
            dev.indexSelect(t.deviceParams(), sel.deviceParams(), indices.deviceParams(), dim)
            acc = TensorValue.from_numpy(x, dev, dtype)
            source = TensorValue.from_numpy(add, dev, dtype)
            dev.indexAdd(source.deviceParams(), acc.deviceParams(), indices.deviceParams(), dim)
            return sel.raw(), acc.numpy()
        got, want = both(b200, ref, run)
        assert np.array_equal(got[0], want[0]), f"indexSelect {DTYPE_NAMES[dtype]} {shape} dim {dim}"
        assert_close(got[1], want[1], dtype, f"indexAdd {DTYPE_NAMES[dtype]} {shape} dim {dim}", scale=np.maximum(1.0, np.abs(want[1]) * 4))
