"""Data-parallel exchange on the GPU through the C ABI: the blocking and the overlapped all-reduce on a communicator of
one rank (stream fork/join, scaling, error behaviour), and - where two GPUs are visible - two ranks as child processes
training the small MLP with both forms of the exchange. Rank failures are not provoked here."""
import os
import subprocess
import sys

import numpy as np
import pytest

from aix_b200 import _capi as C
from aix_b200.tensor import TensorValue

pytestmark = pytest.mark.gpu


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.fixture()
def comm1(b200):
    from aix_b200 import DeviceB200
    b200.commInit(0, 1, DeviceB200.commUniqueId())
    yield b200
    b200.commDestroy()


def test_exchange_needs_a_communicator(b200):
    x = TensorValue.from_numpy(np.ones(16, np.float32), b200)
    with pytest.raises(Exception, match="comm_init"):
        b200.allReduce(x.storage.data, x.size, C.F32, 1.0)
    with pytest.raises(Exception, match="comm_init"):
        b200.allReduceAsync(x.storage.data, x.size, C.F32, 1.0)
    b200.commWait()                                     # nothing in flight: a no-op


def test_single_rank_blocking_sum_and_scale(comm1):
    rng = np.random.default_rng(0)
    host = rng.normal(size=100003).astype(np.float32)
    x = TensorValue.from_numpy(host, comm1)
    comm1.allReduce(x.storage.data, x.size, C.F32, 1.0)
    assert np.array_equal(x.numpy(), host)
    comm1.allReduce(x.storage.data, x.size, C.F32, 0.5)
    assert np.array_equal(x.numpy(), host * np.float32(0.5))
    ints = TensorValue.from_numpy(np.arange(1000, dtype=np.int32), comm1, C.I32)
    comm1.allReduce(ints.storage.data, ints.size, C.I32, 1.0)
    assert np.array_equal(ints.numpy(), np.arange(1000, dtype=np.int32))


def test_single_rank_overlapped_exchange_orders_both_streams(comm1):
    rng = np.random.default_rng(1)
    a = rng.normal(size=(1 << 20)).astype(np.float32)
    b = rng.normal(size=(1 << 20)).astype(np.float32)
    ta, tb = TensorValue.from_numpy(a, comm1), TensorValue.from_numpy(b, comm1)
    g = ta * tb                                          # recorded, not yet launched: the exchange must come after it
    comm1.allReduceAsync(g.storage.data, g.size, C.F32, 1.0)
    other = ta + tb                                      # runs on the device's stream next to the collective
    out = g + other                                      # touches g: the device orders it after g's collective by itself
    assert np.array_equal(out.numpy(), a * b + (a + b))
    # several collectives in flight, consumed one by one in a different order, with an explicit join at the end
    parts = [ta * float(k + 1) for k in range(4)]
    for t in parts:
        comm1.allReduceAsync(t.storage.data, t.size, C.F32, 1.0)
    acc = parts[3] + parts[1]
    comm1.commWait()
    acc = acc + parts[0] + parts[2]
    assert np.allclose(acc.numpy(), a * 10.0, rtol=1e-6)
    # joining one buffer's collective only
    comm1.allReduceAsync(parts[0].storage.data, parts[0].size, C.F32, 1.0)
    comm1.allReduceAsync(parts[1].storage.data, parts[1].size, C.F32, 1.0)
    comm1.commWaitFor(parts[1].storage.data, parts[1].size * 4)
    assert np.allclose((parts[1] * 2.0).numpy(), a * 4.0, rtol=1e-6)
    comm1.commWaitFor(0, 0)                              # nothing to join: a no-op
    # freeing a buffer whose collective is still in flight is safe
    scratch = ta * 2.0
    comm1.allReduceAsync(scratch.storage.data, scratch.size, C.F32, 1.0)
    del scratch
    quarter = ta * 1.0
    comm1.allReduceAsync(quarter.storage.data, quarter.size, C.F32, 0.25)      # any scale: a scaling pass on the side stream
    assert np.array_equal(quarter.numpy(), a * np.float32(0.25))
    # synchronize() joins the side stream on its own
    comm1.allReduceAsync(g.storage.data, g.size, C.F32, 1.0)
    comm1.synchronize()
    assert np.array_equal(g.numpy(), a * b)


def test_single_rank_reduce_scatter_and_all_gather(comm1):
    """One rank: the whole buffer is the rank's own slice - the pair must leave sum x scale there, ordered like any other
    overlapped collective, and refuse counts that do not divide by the number of ranks only when there are several."""
    rng = np.random.default_rng(4)
    host = rng.normal(size=1 << 18).astype(np.float32)
    x = TensorValue.from_numpy(host, comm1)
    y = x * 3.0                                          # pending producer: the collective comes after it
    comm1.reduceScatterAsync(y.storage.data, y.size, C.F32, 0.5)
    z = y + 1.0                                          # touches y: ordered after the collective and its scaling pass
    comm1.allGatherAsync(y.storage.data, y.size, C.F32)
    assert np.array_equal(z.numpy(), host * np.float32(3.0) * np.float32(0.5) + np.float32(1.0))
    assert np.array_equal(y.numpy(), host * np.float32(3.0) * np.float32(0.5))
    assert comm1.commRank() == (0, 1)


def test_sharded_optimizer_on_one_rank_is_the_plain_optimizer(b200):
    from aix_b200.mlp import MlpTrainer
    dims, batch = (64, 128, 32), 48
    plain = MlpTrainer(b200, dims, batch)
    losses = [float(plain.step().value.item()) for _ in range(3)]
    from aix_b200.frontend import ShardedAdam
    again = MlpTrainer(b200, dims, batch)
    again.optimizer = ShardedAdam(again.model.parameters(), 0, 1)
    assert [float(again.step().value.item()) for _ in range(3)] == losses
    for p, q in zip(plain.parameters_numpy(), again.parameters_numpy()):
        assert np.array_equal(p, q)


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_ranks_overlapped_equals_blocking(tmp_path):
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_dp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    results = {}
    for overlap in (0, 1):
        procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(tmp_path), str(overlap), "4"], env=env) for r in range(2)]
        codes = [p.wait(timeout=600) for p in procs]
        assert codes == [0, 0]
        results[overlap] = [np.load(tmp_path / f"rank{r}_{overlap}.npz") for r in range(2)]
    for overlap in (0, 1):
        r0, r1 = results[overlap]
        for k in r0.files:
            if k != "losses":
                assert np.array_equal(r0[k], r1[k]), "ranks diverged"
    # the two forms issue the same collectives on the same data: identical parameters
    for k in results[0][0].files:
        if k != "losses":
            assert np.array_equal(results[0][0][k], results[1][0][k])
    losses = results[1][0]["losses"]
    assert losses[-1] < losses[0]


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_ranks_reproduce_the_single_process_run_on_the_concatenated_batch(tmp_path):
    """Data parallelism must be invisible: two ranks with a batch each, gradients averaged over the ranks, end where one
    process ends that trains on both batches at once (the loss is a mean over the batch, so the gradient of the
    concatenated batch is the average of the two ranks' gradients). f32 tolerance: the sums are formed in a different
    order, and Adam turns a relative perturbation of the gradient into the same relative perturbation of the update."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_dp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    steps = 6
    single = subprocess.Popen([sys.executable, worker, "0", "1", str(tmp_path), "0", str(steps), "2"], env=env)
    assert single.wait(timeout=600) == 0
    want = np.load(tmp_path / "single.npz")
    for mode in ("1", "2", "3"):                          # overlapped all-reduce; sharded optimizer; ... deferred / early updates, gather lane
        procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(tmp_path), mode, str(steps)], env=env) for r in range(2)]
        assert [p.wait(timeout=600) for p in procs] == [0, 0]
        ranks = [np.load(tmp_path / f"rank{r}_{mode}.npz") for r in range(2)]
        for k in want.files:
            if k == "losses":
                continue
            assert np.array_equal(ranks[0][k], ranks[1][k]), f"ranks diverged (exchange {mode})"
            assert np.max(np.abs(ranks[0][k] - want[k])) <= 0.1 * steps * 1e-3, k      # single weights: a fraction of the total movement
            assert np.mean(np.abs(ranks[0][k] - want[k])) <= 2e-6, k                   # the average weight: tightly
        # each rank reports the loss of its own half; their mean is the loss of the concatenated batch
        assert np.allclose(0.5 * (ranks[0]["losses"] + ranks[1]["losses"]), want["losses"], rtol=2e-5)
