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
    for shape, (d0, d1) in [((4, 7), (0, 1)), ((3, 5, 6), (0, 2)), ((3, 5, 6), (1, 2)), ((2, 3, 4, 5), (1, 3)), ((65, 130), (0, 1)),
                             ((257, 100), (0, 1)), ((3, 70, 50), (1, 2)), ((40, 5, 33), (0, 2)), ((2, 33, 3, 64), (1, 3)), ((64, 96, 2), (0, 1)),
                             ((128, 260), (0, 1)), ((3, 68, 72), (1, 2)), ((8, 64, 100), (0, 2))]:      # the last three: rows of whole 16-byte packs
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
def test_contiguous_of_a_large_transposed_matrix(b200, ref, dtype):
    """Large enough for the tiled kernel (ragged tile edges, an offset view), followed and preceded by recorded ops."""
    rng = np.random.default_rng(450 + dtype)
    for rows, cols in [(300, 257), (64, 1030), (1000, 70)]:
        x = values(rng, (rows + 1, cols), dtype)

        def run(dev):
            t = TensorValue.from_numpy(x, dev, dtype)
            u = t + t                                       # a recorded producer
            a = u.transpose(0, 1).contiguous()              # [cols, rows + 1]
            below = TensorValue(t.storage, (rows, cols), t.strides, cols, dtype, dev)      # a view that starts one row in
            b = below.transpose(0, 1).contiguous()          # [cols, rows]
            c = b + b                                       # a recorded consumer
            return a.raw(), b.raw(), c.raw()
        got, want = both(b200, ref, run)
        for g, w in zip(got, want):
            assert np.array_equal(g, w), f"{DTYPE_NAMES[dtype]} {rows}x{cols}"


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_slice_set_tril_triu(b200, ref, dtype):
    rng = np.random.default_rng(500 + dtype)
    for shape, dim, start, end, step in [((8,), 0, 2, 7, 1), ((6, 9), 1, 1, 9, 3), ((6, 9), 0, 0, 6, 2), ((3, 4, 10), 2, 3, 10, 2), ((40, 70), 0, 5, 37, 4),
                                          ((100, 120), 1, 0, 120, 2), ((9, 50, 40), 1, 3, 47, 5), ((200, 64), 0, 10, 190, 1)]:      # large enough for the dense kernel
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
    for shape in [(5, 5), (4, 7), (3, 6, 4), (33, 65), (70, 64), (3, 50, 48), (130, 32)]:      # the last three: whole 16-byte packs per row
        x = values(rng, shape, dtype)
        for diagonal in (-2, 0, 1, 3, -40, 45):
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
    # whole slices as contiguous runs; distinct indices (colliding additions have a test of their own below)
    long_runs = [((200, 64), 0, list(rng.permutation(200)[:100])), ((10, 50, 40), 1, list(rng.permutation(50)[:30])),
                 ((300, 33), 0, list(rng.permutation(300)[:150]))]
    for shape, dim, idx in [((9,), 0, [3, 0, 8, 3]), ((5, 6), 0, [4, 4, 1]), ((5, 6), 1, [0, 5, 2, 2, 3]), ((3, 4, 5), 1, [3, 1]),
                            ((40, 33), 1, list(range(0, 33, 3)))] + long_runs:
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


@pytest.mark.parametrize("dtype", [F32, BF16, I32, I16, U8], ids=lambda d: DTYPE_NAMES[d])
def test_argmax_over_many_blocks_keeps_the_first_maximum(b200, ref, dtype):
    """Sizes that take many CTAs: the two-stage fold must still return the FIRST maximal index
    (aixDeviceCPU.cpp:263-272), also when the maximum occurs thousands of times."""
    rng = np.random.default_rng(900 + dtype)
    for n in (100003, (1 << 21) + 5):
        x = rng.integers(0, 9, n)                       # few distinct values: the maximum 8 appears everywhere
        first = int(np.argmax(x))
        t = TensorValue.from_numpy(x, b200, dtype)
        r = TensorValue.empty((), b200, I32)
        b200.argmax(t.deviceParams(), r.deviceParams())
        assert int(r.numpy()) == first
        oh = TensorValue.empty((n,), b200, I32)
        b200.argmaxIndices(t.deviceParams(), oh.deviceParams())
        got = oh.numpy()
        assert got.sum() == 1 and got[first] == 1
    x = values(rng, (300, 700), dtype)
    got, want = both(b200, ref, lambda dev: _argmax_pair(dev, x, dtype))
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def _argmax_pair(dev, x, dtype):
    t = TensorValue.from_numpy(x, dev, dtype).transpose(0, 1)          # strided source
    r = TensorValue.empty((), dev, I32)
    dev.argmax(t.deviceParams(), r.deviceParams())
    oh = TensorValue.empty(t.shape, dev, I32)
    dev.argmaxIndices(t.deviceParams(), oh.deviceParams())
    return r.numpy(), oh.numpy()


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: DTYPE_NAMES[d])
def test_index_add_with_a_long_index_list_and_collisions(b200, ref, dtype):
    """Few lanes and a long index list take the atomic form: integer results must equal the sequential ones bit for
    bit (wrapping sums commute); floating results within the type's tolerance of the per-add rounding."""
    rng = np.random.default_rng(950 + dtype)
    for shape, dim, count in [((50, 8), 0, 4000), ((3, 64, 4), 1, 1000), ((257,), 0, 5000), ((40, 64), 0, 3000), ((2, 30, 48), 1, 500)]:
        idx = rng.integers(0, shape[dim], count)
        src_shape = list(shape)
        src_shape[dim] = count
        base = values(rng, shape, dtype)
        add = values(rng, src_shape, dtype)
        if dtype in (F32, F64, BF16, F16):
            add = np.round(add / 8.0, 3)                # keep 16-bit running sums in range

        def run(dev):
            acc = TensorValue.from_numpy(base, dev, dtype)
            source = TensorValue.from_numpy(add, dev, dtype)
            indices = TensorValue.from_numpy(idx, dev, I32)
            dev.indexAdd(source.deviceParams(), acc.deviceParams(), indices.deviceParams(), dim)
            return acc.numpy()
        got, want = both(b200, ref, run)
        if dtype in (F32, F64):
            assert_close(got, want, dtype, f"indexAdd {shape}", scale=np.maximum(1.0, np.abs(want)) * 64)
        elif dtype in (BF16, F16):
            # every add rounds to the 16-bit type, in a different order than the sequential loop: compare with the exact sum
            exact = np.array(base, dtype=np.float64)
            np.add.at(np.moveaxis(exact, dim, 0), idx, np.moveaxis(np.array(add, dtype=np.float64), dim, 0))      # a view: adds land in `exact`
            tol = 0.05 * np.maximum(1.0, np.abs(exact)) + 0.3
            assert np.all(np.abs(got - exact) <= tol), f"indexAdd {DTYPE_NAMES[dtype]} {shape}"
        else:
            assert np.array_equal(got, want), f"indexAdd {DTYPE_NAMES[dtype]} {shape}"
