"""Known answers the reference's own tests hold for the front end on this path, replayed through the mirrored front end:
the values of Tests/OptimizerTests.cpp:20-83 (100 steps of SGD and of Adam on m = x*(x*(x+y)/t - y*y) + sin(u)*u, "consistent
with PyTorch" there). On CPU they pin the mirror (run on the reference's CPU device and on the numpy oracle); on the GPU
they pin the device under it. Tolerance: the reference's doctest Approx, 1.19e-5 * (1 + |value|), doubled for the
printed 6-digit constants."""
import numpy as np
import pytest

from aix_b200 import F32
from aix_b200.frontend import SGD, Adam, Tensor
from aix_b200.tensor import TensorValue

EXPECTED = {
    "sgd":  {"lr": 0.001, "values": [2.59247, 4.53346, 4.18035, 4.96434], "grads": [-9.98867, -21.7066, -2.71093, 0.27058]},
    "adam": {"lr": 0.01,  "values": [3.12134, 4.12712, 5.12626, 4.91345], "grads": [-6.25593, -23.6874, -2.66895, 0.00182182]},
}


def train(dev, which):
    x, y, t, u = (Tensor(TensorValue.full(v, (), dev, F32), requireGrad=True) for v in (2.0, 3.0, 4.0, 5.0))
    params = [x, y, t, u]
    optimizer = SGD(params, EXPECTED[which]["lr"]) if which == "sgd" else Adam(params, EXPECTED[which]["lr"])
    for _ in range(100):
        z = x * (x + y) / t - y * y
        m = x * z + u.sin() * u
        optimizer.zeroGrad()
        m.backward()
        optimizer.step()
    return [float(p.value.numpy()) for p in params], [float(p.grad().numpy()) for p in params]


def check(dev, which):
    values, grads = train(dev, which)
    for got, want in zip(values + grads, EXPECTED[which]["values"] + EXPECTED[which]["grads"]):
        assert abs(got - want) <= 2.4e-5 * (1.0 + abs(want)), (which, values, grads)


@pytest.mark.parametrize("which", ["sgd", "adam"])
def test_optimizer_known_answers_on_the_cpu_devices(ref, which):
    from oracle.numpy_oracle import DeviceNumpyOracle
    check(ref, which)
    check(DeviceNumpyOracle(), which)


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["sgd", "adam"])
def test_optimizer_known_answers_on_the_b200(b200, which):
    check(b200, which)


# ---- Tests/DeviceTests.cpp:3478-3500 ("long command batch queue") and :3503-3552 ("loop without sync") -----------------
def long_queue(dev, n=1 << 20):
    ones = np.ones((1, n), np.float32)
    x, y = Tensor(TensorValue.from_numpy(ones, dev)), Tensor(TensorValue.from_numpy(ones, dev))
    z = x + y
    for _ in range(1, 1024):
        z = z + x + y                      # 2047 recorded adds, no synchronisation in between
    dev.synchronize()
    return z.value.numpy()


def xor_training(dev, epochs=1000):
    from aix_b200.frontend import Linear, MSELoss, Sequential, Tanh
    rng = np.random.default_rng(3)         # the reference draws uniform[-1, 1] weights (aix::randn); any seed that converges will do
    model = Sequential(Linear(rng.uniform(-1, 1, (2, 10)).astype(np.float32), rng.uniform(-1, 1, (1, 10)).astype(np.float32), dev), Tanh(),
                       Linear(rng.uniform(-1, 1, (10, 1)).astype(np.float32), rng.uniform(-1, 1, (1, 1)).astype(np.float32), dev))
    inputs = Tensor(TensorValue.from_numpy(np.array([[0, 0], [0, 1], [1, 0], [1, 1]], np.float32), dev))
    targets = Tensor(TensorValue.from_numpy(np.array([[0], [1], [1], [0]], np.float32), dev))
    optimizer, loss_fn = Adam(model.parameters(), 0.01), MSELoss()
    for _ in range(epochs):
        loss = loss_fn(model.forward(inputs), targets)
        optimizer.zeroGrad()
        loss.backward()
        optimizer.step()                   # keeps optimising without synchronising
    loss = loss_fn(model.forward(inputs), targets)
    dev.synchronize()
    return float(loss.value.numpy())


def test_long_queue_and_unsynchronised_training_on_the_numpy_oracle():
    from oracle.numpy_oracle import DeviceNumpyOracle
    dev = DeviceNumpyOracle()
    z = long_queue(dev, n=1 << 12)
    assert z.shape == (1, 1 << 12) and (z == 2048).all()
    assert xor_training(dev) <= 1e-3


@pytest.mark.gpu
def test_long_command_queue_on_the_b200(b200):
    z = long_queue(b200)
    assert z[0, 0] == 2048 and (z == 2048).all()


@pytest.mark.gpu
def test_training_loop_without_synchronisation_on_the_b200(b200):
    assert xor_training(b200) <= 1e-3
