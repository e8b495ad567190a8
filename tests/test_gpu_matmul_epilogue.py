"""Consumers folded into the f32 matmul's epilogue: nn::Linear is matmul(x, W) + b (aixNeuralNetwork.hpp:150-153), usually
followed by tanh. The device holds such a product back until it has seen the recorded ops that follow, and folds
`+ row vector` and `tanh` into the product's kernel as far as the values they consume are dead (temporaries that were
dropped): the kernel then writes one output instead of up to three. Every result must carry the bits the separate kernels
give (same product, same add, same tanh routine), values that are kept alive must still be written, and program order
must hold for ops recorded while the product waits.
"""
import os

import numpy as np
import pytest

from aix_b200 import F32, DeviceB200, TensorValue

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def deep():
    """A second handle on the same GPU that folds the tanh as well: AIXB200_GEMM_EPILOGUE=2, read when a device is created.
    The default (1) folds the add only - measured, the tanh is cheaper as a kernel of its own."""
    old = os.environ.get("AIXB200_GEMM_EPILOGUE")
    os.environ["AIXB200_GEMM_EPILOGUE"] = "2"
    try:
        dev = DeviceB200(0)
    finally:
        if old is None: os.environ.pop("AIXB200_GEMM_EPILOGUE")
        else: os.environ["AIXB200_GEMM_EPILOGUE"] = old
    yield dev
    dev.synchronize()
    dev.close()


def folded(b200):
    return b200.stats()["matmul_consumers_folded"]


def operands(b200, m, k, n, seed):
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    w = (rng.normal(0, 1, (k, n)) / np.sqrt(k)).astype(np.float32)
    b = rng.normal(0, 0.5, (1, n)).astype(np.float32)
    return x, w, b, TensorValue.from_numpy(x, b200), TensorValue.from_numpy(w, b200), TensorValue.from_numpy(b, b200)


def separate(b200, tx, tw, tb):
    """The same three results from three launches: a synchronisation after each call keeps anything from being folded."""
    mm = tx.matmul(tw)
    b200.synchronize()
    s = mm + tb
    b200.synchronize()
    t = s.tanh()
    b200.synchronize()
    return mm.numpy(), s.numpy(), t.numpy()


@pytest.mark.parametrize("m,k,n", [(256, 128, 256), (512, 256, 384), (300, 100, 200), (1024, 1024, 1024), (257, 64, 68), (4096, 320, 512)])
def test_linear_tanh_is_one_launch_with_the_bits_of_three(deep, ref, m, k, n):
    b200 = deep
    x, w, b, tx, tw, tb = operands(b200, m, k, n, m + n)
    want_mm, want_s, want_t = separate(b200, tx, tw, tb)
    before, launches = folded(b200), b200.stats()["total_kernel_launches"]
    t = (tx.matmul(tw) + tb).tanh()     # the product and the sum are temporaries: dead by the time the product is launched
    b200.synchronize()
    assert folded(b200) == before + 2, "the add and the tanh ran inside the product's kernel"
    assert b200.stats()["total_kernel_launches"] - launches == 1, "one product, no elementwise kernel"
    assert np.array_equal(t.numpy(), want_t)
    exact = x.astype(np.float64) @ w.astype(np.float64) + b.astype(np.float64)
    assert np.max(np.abs(want_s - exact)) <= 1e-5 * np.max(np.abs(exact))
    assert np.max(np.abs(t.numpy() - np.tanh(exact))) <= 2e-5
    # and against the reference's CPU device on a slab of rows
    rows = slice(0, 8)
    rx, rw, rb = TensorValue.from_numpy(x[rows], ref), TensorValue.from_numpy(w, ref), TensorValue.from_numpy(b, ref)
    cpu = (rx.matmul(rw) + rb).tanh().numpy()
    assert np.max(np.abs(t.numpy()[rows] - cpu)) <= 2e-5
    # everything kept alive, as autograd keeps it: nothing is folded, every value is written
    before = folded(b200)
    mm = tx.matmul(tw)
    s = mm + tb
    t = s.tanh()
    b200.synchronize()
    assert folded(b200) == before
    assert np.array_equal(mm.numpy(), want_mm) and np.array_equal(s.numpy(), want_s) and np.array_equal(t.numpy(), want_t)


def test_by_default_the_add_is_folded_when_no_recorded_op_consumes_the_sum(b200):
    """Measured: a recorded consumer runs in one generated kernel together with the add, so folding the add there saves no
    pass over memory; folding pays when the sum goes straight to a matmul, a reduction kernel or the host."""
    x, w, b, tx, tw, tb = operands(b200, 512, 256, 384, 11)
    want_mm, want_s, want_t = separate(b200, tx, tw, tb)
    before, launches = folded(b200), b200.stats()["total_kernel_launches"]
    t = (tx.matmul(tw) + tb).tanh()
    b200.synchronize()
    assert folded(b200) == before
    assert b200.stats()["total_kernel_launches"] - launches == 2, "the product, then add + tanh as one generated kernel"
    assert np.array_equal(t.numpy(), want_t)
    before, launches = folded(b200), b200.stats()["total_kernel_launches"]
    s = tx.matmul(tw) + tb
    b200.synchronize()
    assert folded(b200) == before + 1
    assert b200.stats()["total_kernel_launches"] - launches == 1
    assert np.array_equal(s.numpy(), want_s)
    before = folded(b200)
    y = (tx.matmul(tw) + tb).matmul(TensorValue.from_numpy(np.eye(384, dtype=np.float32), b200))      # straight into the next product
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.max(np.abs(y.numpy() - want_s)) <= 1e-5 * np.max(np.abs(want_s))


def test_bias_on_the_left_and_bias_only(b200, deep):
    x, w, b, tx, tw, tb = operands(b200, 512, 128, 256, 5)
    want_mm, want_s, want_t = separate(b200, tx, tw, tb)
    before = folded(b200)
    s = tb + tx.matmul(tw)              # row vector first
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(s.numpy(), want_s)
    b200 = deep
    x, w, b, tx, tw, tb = operands(b200, 512, 128, 256, 5)
    before = folded(b200)
    s = tx.matmul(tw) + tb
    u = s * 2.0                         # the sum's first consumer is not a tanh: the product is launched with the add folded
    t = s.tanh()
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(s.numpy(), want_s)
    assert np.array_equal(u.numpy(), want_s * np.float32(2.0))
    assert np.array_equal(t.numpy(), want_t)
    before = folded(b200)
    s = tx.matmul(tw) + tb
    t = s.tanh()                        # the sum stays alive: only the add is folded, the tanh runs as a kernel
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(s.numpy(), want_s) and np.array_equal(t.numpy(), want_t)


def test_other_first_consumers_leave_the_product_alone(b200):
    x, w, b, tx, tw, tb = operands(b200, 512, 128, 256, 6)
    want_mm, want_s, want_t = separate(b200, tx, tw, tb)
    before = folded(b200)
    mm = tx.matmul(tw)
    d = mm * mm                         # not `+ row vector`
    s = mm + tb
    del mm
    b200.synchronize()
    assert folded(b200) == before
    assert np.array_equal(d.numpy(), want_mm * want_mm)
    assert np.array_equal(s.numpy(), want_s)
    full = TensorValue.from_numpy(np.broadcast_to(b, (512, 256)).copy(), b200)
    s = tx.matmul(tw) + full            # a full matrix, not a row vector
    b200.synchronize()
    assert folded(b200) == before
    assert np.array_equal(s.numpy(), want_s)
    col = TensorValue.from_numpy(np.ones((512, 1), dtype=np.float32), b200)
    s = tx.matmul(tw) + col             # a column vector
    b200.synchronize()
    assert folded(b200) == before
    assert np.array_equal(s.numpy(), want_mm + np.float32(1.0))
    mm = tx.matmul(tw)
    s = mm + tb
    e = mm * 0.5                        # the product is read again after its add: it must be written
    del mm
    t = s.tanh()
    del s
    b200.synchronize()
    assert folded(b200) == before
    assert np.array_equal(e.numpy(), want_mm * np.float32(0.5)) and np.array_equal(t.numpy(), want_t)


def test_program_order_around_a_waiting_product(deep):
    b200 = deep
    x, w, b, tx, tw, tb = operands(b200, 512, 128, 256, 7)
    want_mm, want_s, want_t = separate(b200, tx, tw, tb)
    bias = TensorValue.from_numpy(b, b200)
    weights = TensorValue.from_numpy(w, b200)
    before = folded(b200)
    mm = tx.matmul(weights)
    s = mm + bias
    bias += 1.0                         # written after the add was recorded: the add still sees the old bias
    weights *= 0.0                      # ... and the product the old weights
    mm *= 2.0                           # ... and the add saw the product before this
    t = s.tanh()
    b200.synchronize()
    assert folded(b200) == before
    assert np.array_equal(s.numpy(), want_s)
    assert np.array_equal(t.numpy(), want_t)
    assert np.array_equal(mm.numpy(), want_mm * np.float32(2.0))
    assert np.array_equal(bias.numpy(), b + np.float32(1.0))
    assert not weights.numpy().any()
    # the same with the product dropped: the add is folded and reads bias and weights as they were
    bias = TensorValue.from_numpy(b, b200)
    weights = TensorValue.from_numpy(w, b200)
    before = folded(b200)
    s = tx.matmul(weights) + bias
    bias += 1.0
    weights *= 0.0
    t = s.tanh()
    del s
    z = TensorValue.full(3.0, (1000,), b200, F32)       # an unrelated fill does not end the wait
    b200.synchronize()
    assert folded(b200) == before + 2
    assert np.array_equal(t.numpy(), want_t)
    assert np.array_equal(bias.numpy(), b + np.float32(1.0))
    assert not weights.numpy().any()
    assert (z.numpy() == 3.0).all()
    assert not tx.matmul(weights).numpy().any(), "the form prepared for the waiting product is not reused after the in-place update"
    # a reduction recorded behind the folded add
    before = folded(b200)
    s = tx.matmul(tw) + tb
    total = s.sum()
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(s.numpy(), want_s)
    assert abs(float(total.numpy()) - want_s.astype(np.float64).sum()) <= 1e-5 * np.abs(want_s).sum()


@pytest.mark.parametrize("with_tanh", [False, True], ids=["sum", "tanh"])
def test_the_next_product_finds_the_maximum_the_epilogue_left(b200, deep, with_tanh):
    """Two layers: the second product's left operand is the first one's folded output; its max|x| comes from the first
    product's epilogue once the size is known as an operand size (from the second step on)."""
    dev = deep if with_tanh else b200
    rng = np.random.default_rng(9)
    m, k = 1024, 1024
    x = TensorValue.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32), dev)
    w1 = TensorValue.from_numpy((rng.normal(0, 1, (k, k)) / 32).astype(np.float32), dev)
    w2 = TensorValue.from_numpy((rng.normal(0, 1, (k, k)) / 32).astype(np.float32), dev)
    b1 = TensorValue.from_numpy(rng.normal(0, 0.5, (1, k)).astype(np.float32), dev)
    results = []
    for step in range(3):
        known, before = dev.stats()["prepared_operand_max_known"], folded(dev)
        h = (x.matmul(w1) + b1).tanh() if with_tanh else x.matmul(w1) + b1
        y = h.matmul(w2)
        dev.synchronize()
        assert folded(dev) == before + (2 if with_tanh else 1)
        results.append((h.numpy(), y.numpy(), dev.stats()["prepared_operand_max_known"] - known))
    assert results[2][2] >= 1, "the folded output's maximum was left by the epilogue"
    exact_h = x.numpy().astype(np.float64) @ w1.numpy().astype(np.float64) + b1.numpy().astype(np.float64)
    if with_tanh: exact_h = np.tanh(exact_h)
    exact_y = exact_h @ w2.numpy().astype(np.float64)
    for h, y, _ in results:
        assert np.array_equal(h, results[0][0])
        assert np.max(np.abs(y - exact_y)) <= 1e-5 * np.max(np.abs(exact_y))
        assert np.array_equal(y, results[0][1]), "the scale taken from the epilogue's maximum is the one the max pass finds"


def test_a_dead_product_lands_in_the_zero_filled_buffer_it_is_accumulated_into(b200):
    """`grad += x^T . G` after zeroGrad(): the fill and the add disappear, the product is written into the gradient buffer."""
    x, w, b, tx, tw, tb = operands(b200, 512, 256, 384, 21)
    want_mm, _, _ = separate(b200, tx, tw, tb)
    before, launches = folded(b200), b200.stats()["total_kernel_launches"]
    g = TensorValue.full(0.0, (512, 384), b200)
    g += tx.matmul(tw)
    b200.synchronize()
    assert folded(b200) == before + 1
    assert b200.stats()["total_kernel_launches"] - launches == 1, "the product alone: no fill kernel, no add kernel"
    assert np.array_equal(g.numpy(), want_mm)
    g += tx.matmul(tw)                  # no fill recorded any more: an ordinary accumulation
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(g.numpy(), want_mm + want_mm)
    g = TensorValue.full(0.5, (512, 384), b200)     # not zero
    g += tx.matmul(tw)
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(g.numpy(), np.float32(0.5) + want_mm)
    g = TensorValue.full(0.0, (512, 384), b200)
    mm = tx.matmul(tw)                  # the product stays alive: it must be written itself
    g += mm
    b200.synchronize()
    assert folded(b200) == before + 1
    assert np.array_equal(g.numpy(), want_mm) and np.array_equal(mm.numpy(), want_mm)
    g = TensorValue.full(0.0, (512, 384), b200)
    g += tx.matmul(tw)
    h = g * 2.0                         # a reader of the target recorded while the product waits
    b200.synchronize()
    assert np.array_equal(g.numpy(), want_mm) and np.array_equal(h.numpy(), want_mm * np.float32(2.0))
