"""Data-parallel host logic on CPU: two gloo ranks, each with a CPU device (the numpy oracle) and the mirrored front
end, exchange gradients through the same `all_reduce_gradients` call the GPU path uses (the device's allReduce is
served by gloo here instead of NCCL). After three Adam steps on per-rank batches every rank must hold the parameters
a single process gets from the concatenated batch, and both ranks must agree bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aix_b200 import _capi as C
from aix_b200.mlp import MlpTrainer, synthetic_batch, xavier_parameters
from aix_b200.frontend import Tensor
from aix_b200.tensor import TensorValue
from oracle.numpy_oracle import DeviceNumpyOracle

DIMS = (8, 16, 16, 4)
BATCH = 6
STEPS = 3


class GlooDevice(DeviceNumpyOracle):
    """CPU device whose allReduce goes through torch.distributed (gloo): sum over ranks, then scale."""

    def allReduce(self, data, count, dtype, scale=1.0):
        assert dtype == C.F32
        view = self._raw(data, dtype, count)
        t = torch.from_numpy(view.copy())
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        view[:] = (t.numpy() * np.float32(scale)).astype(np.float32)

    # A CPU device has one "stream": the overlapped form degenerates to the blocking one, which still exercises the
    # hook order (one collective per parameter, issued in the same order on every rank).
    def allReduceAsync(self, data, count, dtype, scale=1.0):
        self.async_calls = getattr(self, "async_calls", 0) + 1
        self.allReduce(data, count, dtype, scale)

    def _write(self, p, values):
        """The sharded optimizer updates a slice of a parameter in place, i.e. it hands the device a RESULT view with an
        offset. The B200 device writes through the result view; the reference's CPU device writes res[i] from the
        storage base whatever the view's offset (aixDeviceCPU.cpp:36-40), which is why this test double honours the
        offset of dense results (identical for offset 0, the only case the reference's own callers produce)."""
        self._raw(p.data, p.dtype, p.offset + len(values))[p.offset:] = values

    def reduceScatterAsync(self, data, count, dtype, scale=1.0):
        """Slice `rank` of the buffer receives the scaled sum; the other slices are scribbled over on purpose - nothing
        may read them before the all-gather."""
        self.scatter_calls = getattr(self, "scatter_calls", 0) + 1
        view = self._raw(data, dtype, count)
        t = torch.from_numpy(view.copy())
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        n, r = count // dist.get_world_size(), dist.get_rank()
        reduced = (t.numpy() * np.float32(scale)).astype(np.float32)
        view[:] = np.float32(np.nan)
        view[r * n:(r + 1) * n] = reduced[r * n:(r + 1) * n]

    def allGatherAsync(self, data, count, dtype):
        self.gather_calls = getattr(self, "gather_calls", 0) + 1
        view = self._raw(data, dtype, count)
        n, r = count // dist.get_world_size(), dist.get_rank()
        parts = [torch.empty(n, dtype=torch.float32) for _ in range(dist.get_world_size())]
        dist.all_gather(parts, torch.from_numpy(view[r * n:(r + 1) * n].copy()))
        view[:] = torch.cat(parts).numpy()

    def commWait(self):
        self.waits = getattr(self, "waits", 0) + 1

    def commWaitFor(self, data, nbytes):
        self.joins = getattr(self, "joins", 0) + 1


def set_batch(trainer, dev, x, y):
    trainer.x = Tensor(TensorValue.from_numpy(x, dev))
    trainer.y = Tensor(TensorValue.from_numpy(y, dev))


def worker(rank, world, port, out_dir, overlap=True, sharded=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = GlooDevice()
    weights, biases = xavier_parameters(DIMS, seed=0)
    deferred = sharded == "deferred"               # updates of the late layers inside the next forward pass, of the early ones inside backward
    trainer = MlpTrainer(dev, DIMS, BATCH, rank=rank, world_size=world, weights=weights, biases=biases, overlap=overlap, sharded=bool(sharded),
                         deferred=deferred, early=deferred)
    x, y = synthetic_batch(DIMS, BATCH, rank)
    set_batch(trainer, dev, x, y)
    for _ in range(STEPS):
        trainer.step()
    if sharded:
        if deferred:
            # the deferred optimizer owes the last step's updates of the later half of the modules until the next forward pass or finish()
            owed = sum(len(m.parameters()) for m in [m for m in trainer.model.modules if m.parameters()][trainer.optimizer._eager:])
            assert dev.gather_calls == STEPS * len(trainer.model.parameters()) - owed
        trainer.optimizer.finish()
        # one reduce-scatter, one join and one all-gather per parameter and step; the optimizer state is 1/world of a replica's
        count = STEPS * len(trainer.model.parameters())
        assert dev.scatter_calls == count == dev.gather_calls == dev.joins and not hasattr(dev, "async_calls")
        assert sum(m.size for m in trainer.optimizer.m) * world == sum(p.value.size for p in trainer.model.parameters())
    elif overlap:
        # one collective and one join per parameter and step; no global join when the optimizer is attached
        assert dev.async_calls == STEPS * len(trainer.model.parameters()) == dev.joins and not hasattr(dev, "waits")
    else:
        assert not hasattr(dev, "async_calls")
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), *trainer.parameters_numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("overlap,sharded", [(True, False), (False, False), (True, "eager"), (True, "deferred")],
                         ids=["overlapped", "after_backward", "sharded_optimizer", "sharded_optimizer_deferred_and_early"])
def test_two_ranks_equal_one_process_on_the_global_batch(tmp_path, overlap, sharded):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(worker, args=(2, port, str(tmp_path), overlap, sharded), nprocs=2, join=True)
    r0 = np.load(tmp_path / "rank0.npz")
    r1 = np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), "ranks diverged"

    dev = DeviceNumpyOracle()
    weights, biases = xavier_parameters(DIMS, seed=0)
    single = MlpTrainer(dev, DIMS, 2 * BATCH, weights=weights, biases=biases)
    xs, ys = zip(*(synthetic_batch(DIMS, BATCH, r) for r in range(2)))
    set_batch(single, dev, np.concatenate(xs), np.concatenate(ys))
    for _ in range(STEPS):
        single.step()
    for got, want in zip((r0[k] for k in r0.files), single.parameters_numpy()):
        assert np.allclose(got, want, rtol=1e-4, atol=2e-5), np.max(np.abs(got - want))


def mean_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aix_b200.frontend import global_mean
    dev = GlooDevice()
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (12, 40)).astype(np.float32)           # every rank draws the same matrix and keeps its own rows
    g = rng.uniform(0.5, 1.5, 40).astype(np.float32)
    rows = x.shape[0] // world
    tx, tg = TensorValue.from_numpy(x[rank * rows:(rank + 1) * rows], dev), TensorValue.from_numpy(g, dev)
    y = tx * tg
    np.savez(os.path.join(out_dir, f"mean{rank}.npz"), mean=global_mean(y, world).numpy(), row_sum=y.sum(1).numpy(), row_max=y.max(1).numpy())
    dist.destroy_process_group()


def test_row_sharded_reductions_need_one_scalar_exchange(tmp_path):
    """Configuration 1 split by rows over two ranks: row sums and row maxima are local, the global mean takes one scalar
    all-reduce and equals the single-process mean."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(mean_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (12, 40)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, 40).astype(np.float32)
    dev = DeviceNumpyOracle()
    y = TensorValue.from_numpy(x, dev) * TensorValue.from_numpy(g, dev)
    parts = [np.load(tmp_path / f"mean{r}.npz") for r in range(2)]
    assert np.array_equal(parts[0]["mean"], parts[1]["mean"])
    assert abs(float(parts[0]["mean"]) - float(y.mean().numpy())) <= 1e-6 * max(1.0, abs(float(y.mean().numpy())))
    assert np.array_equal(np.concatenate([p["row_sum"] for p in parts]), y.sum(1).numpy())
    assert np.array_equal(np.concatenate([p["row_max"] for p in parts]), y.max(1).numpy())


def test_shards_are_disjoint_and_deterministic():
    a0, _ = synthetic_batch(DIMS, BATCH, rank=0)
    a1, _ = synthetic_batch(DIMS, BATCH, rank=1)
    b0, _ = synthetic_batch(DIMS, BATCH, rank=0)
    assert np.array_equal(a0, b0) and not np.array_equal(a0, a1)
    w0, _ = xavier_parameters(DIMS, seed=0)
    w1, _ = xavier_parameters(DIMS, seed=0)
    assert all(np.array_equal(x, y) for x, y in zip(w0, w1))          # identical replicas on every rank


def test_exchange_refuses_a_second_contribution_in_flight():
    from aix_b200.frontend import GradientExchange

    class Recorder(DeviceNumpyOracle):
        def allReduceAsync(self, data, count, dtype, scale=1.0): pass
        def commWait(self): pass

    dev = Recorder()
    w = Tensor(TensorValue.from_numpy(np.ones((2, 2), np.float32), dev), requireGrad=True)
    exchange = GradientExchange(dev, [w], world_size=2)
    y = (w + w.tanh()).sum()                              # two separate contributions to w
    with pytest.raises(RuntimeError, match="second gradient contribution"):
        y.backward()
    exchange.finish()
    exchange.detach()
    assert w.node.gradReadyHook is None
