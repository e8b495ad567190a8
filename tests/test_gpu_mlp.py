"""MLP training through the mirrored front end on the B200 device against the reference's own front end on its CPU
device (scaled-down widths so the CPU finishes in seconds), plus piecewise checks at the full layer width."""
import numpy as np
import pytest

from aix_b200 import F32, TensorValue
from aix_b200.mlp import MlpTrainer, synthetic_batch, xavier_parameters

pytestmark = pytest.mark.gpu


def test_loss_curve_and_parameters_follow_the_reference_front_end(b200, ref):
    dims = (64, 256, 256, 256, 64)
    batch, steps = 128, 10
    weights, biases = xavier_parameters(dims, seed=0)
    x, y = synthetic_batch(dims, batch)
    trainer = MlpTrainer(b200, dims, batch, weights=[w.copy() for w in weights], biases=[b.copy() for b in biases])
    got_losses = np.array([float(trainer.step().value.item()) for _ in range(steps)])
    ref_w, ref_b = [w.copy() for w in weights], [b.copy() for b in biases]
    want_losses, _ = ref.mlp_train_f32(list(dims), ref_w, ref_b, x, y, steps, lr=1e-3)
    assert np.allclose(got_losses, want_losses, rtol=2e-5), (got_losses, want_losses)
    params = trainer.parameters_numpy()
    for i in range(4):
        # Adam moves every weight by about lr per step whatever the gradient's size, and for weights whose gradient is
        # rounding noise the direction itself is noise: bound single weights by a fraction of the total movement
        # (steps * lr = 1e-2) and the average weight tightly.
        for got, want in ((params[2 * i], ref_w[i]), (params[2 * i + 1], ref_b[i])):
            assert np.max(np.abs(got - want)) <= 0.1 * steps * 1e-3
            assert np.mean(np.abs(got - want)) <= 2e-6


def test_full_width_step_runs_and_reduces_the_loss(b200):
    trainer = MlpTrainer(b200, batch=512)
    losses = [float(trainer.step().value.item()) for _ in range(4)]
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]
    stats = b200.stats()
    assert stats["static_kernel_launches"] > 0 and stats["fused_kernels"] > 0
