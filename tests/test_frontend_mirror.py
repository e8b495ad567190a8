"""The Python mirror of the reference's front end (aix_b200/frontend.py) must issue the same device work as the
reference's own aix::Tensor / nn / optim classes. Proof: run the mirror on a CPU device and compare with the golden
record of the reference front end training the same tiny MLP (tests/golden/make_golden.py, "mlp/*"): losses and
trained parameters must agree to the last bit on the reference's CPU device, and within float rounding of the
transcendental functions on the numpy oracle."""
import os

import numpy as np
import pytest

from aix_b200 import F32, TensorValue
from aix_b200.frontend import Adam, Linear, MSELoss, Sequential, Tanh, Tensor
from oracle.numpy_oracle import DeviceNumpyOracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_ops.npz")


def train(dev, golden, steps=3):
    layers = []
    for i in range(3):
        layers.append(Linear(golden[f"mlp/w{i}_init"], golden[f"mlp/b{i}_init"], dev))
        if i < 2:
            layers.append(Tanh())
    model = Sequential(*layers)
    x = Tensor(TensorValue.from_numpy(golden["mlp/x"], dev))
    y = Tensor(TensorValue.from_numpy(golden["mlp/y"], dev))
    opt = Adam(model.parameters(), lr=1e-3)
    loss_fn = MSELoss()
    losses = []
    for _ in range(steps):
        pred = model.forward(x)
        loss = loss_fn(pred, y)
        opt.zeroGrad()
        loss.backward()
        opt.step()
        losses.append(float(loss.value.item()))
    params = [p.value.numpy() for p in model.parameters()]
    return np.array(losses, dtype=np.float32), params


def test_mirror_on_reference_cpu_device_is_bit_identical_to_reference_front_end(ref):
    golden = np.load(GOLDEN)
    losses, params = train(ref, golden)
    assert np.array_equal(losses, golden["mlp/losses"])
    for i in range(3):
        assert np.array_equal(params[2 * i], golden[f"mlp/w{i}_final"])
        assert np.array_equal(params[2 * i + 1], golden[f"mlp/b{i}_final"])


def test_mirror_on_numpy_oracle_matches_reference_front_end():
    golden = np.load(GOLDEN)
    losses, params = train(DeviceNumpyOracle(), golden)
    assert np.allclose(losses, golden["mlp/losses"], rtol=2e-6, atol=0)
    for i in range(3):
        assert np.allclose(params[2 * i], golden[f"mlp/w{i}_final"], rtol=1e-5, atol=1e-7)
        assert np.allclose(params[2 * i + 1], golden[f"mlp/b{i}_final"], rtol=1e-5, atol=1e-7)


def test_training_step_issues_the_documented_op_stream(dry):
    """4 Linear + 3 Tanh: per parameter Adam issues 14 arithmetic calls and 8 scalar fills (22 device calls) - and the
    planner turns the 168 optimizer ops into one kernel per distinct parameter size."""
    rng = np.random.default_rng(0)
    dims = [16, 32, 32, 32, 16]
    layers = []
    for i in range(4):
        layers.append(Linear(rng.normal(0, 0.1, (dims[i], dims[i + 1])).astype(np.float32), np.zeros(dims[i + 1], dtype=np.float32), dry))
        if i < 3:
            layers.append(Tanh())
    model = Sequential(*layers)
    x = Tensor(TensorValue.from_numpy(rng.normal(0, 1, (8, 16)).astype(np.float32), dry))
    y = Tensor(TensorValue.from_numpy(rng.normal(0, 1, (8, 16)).astype(np.float32), dry))
    opt = Adam(model.parameters())
    loss_fn = MSELoss()
    for _ in range(2):                   # the first step also creates the gradient buffers
        loss = loss_fn(model.forward(x), y)
        opt.zeroGrad()
        loss.backward()
        dry.synchronize()
        before = dry.stats()
        opt.step()
        dry.synchronize()
        after = dry.stats()
    assert after["ops_recorded"] - before["ops_recorded"] == 8 * 22
    # parameter sizes: 16x32, 32x32 (twice), 32x16 (= 16x32 elements), 1x32 (three times), 1x16
    assert after["fused_kernels"] - before["fused_kernels"] <= 4
    assert after["fills_absorbed"] - before["fills_absorbed"] == 8 * 8
