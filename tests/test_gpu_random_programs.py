"""Differential test of the lazy recorder: seeded random programs - elementwise ops on full tensors, row / column
broadcasts and transposed views, in-place updates, full sums and maxima in the middle of chains, scalars derived from
reductions fed back into later ops, tensors dropped while work is pending - run on the B200 device and on the reference's
CPU device; every tensor still alive at the end must agree. The reference evaluates each call at once, so any ordering,
forwarding or elision mistake of the planner shows up as a numeric difference."""
import numpy as np
import pytest

from aix_b200 import F32, TensorValue
from conftest import assert_close

pytestmark = pytest.mark.gpu

ROWS, COLS = 37, 129            # ragged on purpose: packs, tails and broadcasts all take their slow edges


def run_program(dev, seed):
    rng = np.random.default_rng(seed)
    data = np.random.default_rng(1000 + seed)
    full = [TensorValue.from_numpy(data.uniform(-1, 1, (ROWS, COLS)).astype(np.float32), dev) for _ in range(3)]
    rowv = TensorValue.from_numpy(data.uniform(-1, 1, (1, COLS)).astype(np.float32), dev)
    colv = TensorValue.from_numpy(data.uniform(-1, 1, (ROWS, 1)).astype(np.float32), dev)
    square = TensorValue.from_numpy(data.uniform(-1, 1, (COLS, ROWS)).astype(np.float32), dev)
    scalars = []
    for _ in range(int(rng.integers(15, 40))):
        kind = int(rng.integers(0, 12))
        i, j = int(rng.integers(0, len(full))), int(rng.integers(0, len(full)))
        a, b = full[i], full[j]
        if kind == 0:   full.append((a + b).tanh())
        elif kind == 1: full.append(a * b - a)
        elif kind == 2: full.append((a * rowv.broadcastTo((ROWS, COLS)) + colv.broadcastTo((ROWS, COLS))).sin())
        elif kind == 3: full.append(a - square.transpose(0, 1) * 0.5)
        elif kind == 4: a += b * 0.25                                     # in place, possibly with itself as operand
        elif kind == 5: a *= (b * b + 1.0).sqrt() * 0.5
        elif kind == 6: scalars.append(a.sum())
        elif kind == 7: scalars.append((a * b).max())
        elif kind == 8 and scalars:                                       # a reduction's result fed back as a broadcast scalar
            s = scalars[int(rng.integers(0, len(scalars)))]
            full.append((a + s.broadcastTo((ROWS, COLS)) * (1.0 / (ROWS * COLS))).cos())
        elif kind == 9 and len(full) > 3: full.pop(int(rng.integers(3, len(full))))      # dropped while ops are pending
        elif kind == 10: full.append((-a).exp() * 0.1 + b / (a * a + 1.0))
        elif kind == 11:
            t = a * 2.0                                                     # dead after the reductions: never stored
            scalars.append(t.sum()); scalars.append(t.max())
        if len(full) > 12: full.pop(3)
    return [t.numpy() for t in full], [float(s.numpy()) for s in scalars]


@pytest.mark.parametrize("seed", range(24))
def test_random_program_matches_the_cpu_device(b200, ref, seed):
    got_t, got_s = run_program(b200, seed)
    want_t, want_s = run_program(ref, seed)
    assert len(got_t) == len(want_t) and len(got_s) == len(want_s)
    for k, (g, w) in enumerate(zip(got_t, want_t)):
        assert np.isfinite(w).all()
        assert_close(g, w, F32, f"seed {seed}: tensor {k}", scale=max(1.0, float(np.abs(w).max())) * 4.0)
    for k, (g, w) in enumerate(zip(got_s, want_s)):
        assert abs(g - w) <= 4e-5 * max(1.0, abs(w), ROWS * COLS * 0.25), f"seed {seed}: scalar {k}: {g} vs {w}"


def test_fills_kept_across_flushes_land_in_program_order(b200, ref):
    """A fill whose buffer nothing uses yet stays recorded over later flushes. Whatever comes next - an accumulation, a
    read through another call, a second fill, a host read, a deallocation - must see it exactly where it was issued."""
    import numpy as np
    from aix_b200 import F32, TensorValue
    rng = np.random.default_rng(77)
    a = rng.normal(0, 1, (256, 192)).astype(np.float32)
    b = rng.normal(0, 1, (192, 256)).astype(np.float32)
    outs = []
    for dev in (b200, ref):
        ta, tb = TensorValue.from_numpy(a, dev), TensorValue.from_numpy(b, dev)
        g1 = TensorValue.full(0.0, (256, 256), dev)          # accumulated into after two matmuls
        g2 = TensorValue.full(5.0, (256, 256), dev)          # read by a reduction (an immediate call) later
        g3 = TensorValue.full(1.0, (256, 256), dev)          # overwritten by a second fill, then read on the host
        g4 = TensorValue.full(9.0, (256, 256), dev)          # dropped without ever being used
        c = ta.matmul(tb)
        d = c.matmul(ta.matmul(tb))
        g1 += d
        g1 += c
        del g4
        s = g2.sum(0)
        g3.fill(2.0)
        e = ta.matmul(tb)
        g2 += e
        outs.append([g1.numpy(), s.numpy(), g3.numpy(), g2.numpy()])
    from conftest import assert_close
    for k, what in enumerate(("accumulated", "column sums of a filled buffer", "refilled", "filled then accumulated")):
        # matmul results are compared norm-wise (the CPU device's own sequential f32 dot products carry that much error)
        assert_close(outs[0][k], outs[1][k], F32, what, scale=float(np.max(np.abs(outs[1][k]))) if k in (0, 3) else None)
