"""Child process of tests/test_gpu_comm.py: one data-parallel rank on its own GPU.

    python tests/_dp_worker.py <rank> <world> <dir> <exchange 0|1|2|3> <steps> [<ranks whose batches one process concatenates>]

exchange: 0 = all-reduces after backward, 1 = all-reduces started inside backward, 2 = sharded optimizer (reduce-scatter,
per-rank slice of Adam, all-gather; all collectives on one communicator), 3 = the same with the all-gathers on a communicator
of their own (the default), the late layers' updates deferred into the next forward pass and the early layers' moved into backward.

Rank 0 publishes the communicator id through a file in <dir>; every rank trains the small MLP and writes its parameters
and losses to <dir>/rank<r>_<overlap>.npz. With world = 1 and the last argument R, the single process trains on the
concatenation of the batches ranks 0 .. R-1 would have drawn (the single-process result the data-parallel run must
reproduce) and writes <dir>/single.npz."""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from aix_b200 import DeviceB200                      # noqa: E402
from aix_b200.mlp import MlpTrainer, synthetic_batch  # noqa: E402

DIMS = (256, 512, 512, 128)
BATCH = 384


def main():
    rank, world, out_dir, mode, steps = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4]), int(sys.argv[5])
    overlap, sharded, deferred = mode >= 1, mode >= 2, mode == 3
    if mode == 2:
        os.environ["AIXB200_COMM_GATHER_LANE"] = "0"        # mode 2: every collective on one communicator; mode 3: all-gathers on their own (default)
    concat = int(sys.argv[6]) if len(sys.argv) > 6 else 0
    if world == 1 and concat > 1:
        parts = [synthetic_batch(DIMS, BATCH, r) for r in range(concat)]
        data = (np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts]))
        dev = DeviceB200(rank)
        trainer = MlpTrainer(dev, DIMS, data=data)
        losses = [float(trainer.step().value.numpy()) for _ in range(steps)]
        dev.synchronize()
        np.savez(os.path.join(out_dir, "single.npz"), *trainer.parameters_numpy(), losses=np.array(losses))
        dev.close()
        return
    id_path = os.path.join(out_dir, f"comm_id_{mode}")
    if rank == 0:
        unique = DeviceB200.commUniqueId()
        with open(id_path + ".tmp", "wb") as f:
            f.write(unique)
        os.replace(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 120
        while not os.path.exists(id_path):
            if time.time() > deadline:
                raise SystemExit("rank 0 never published the communicator id")
            time.sleep(0.05)
        with open(id_path, "rb") as f:
            unique = f.read()
    dev = DeviceB200(rank)
    dev.commInit(rank, world, unique)
    trainer = MlpTrainer(dev, DIMS, BATCH, rank=rank, world_size=world, overlap=overlap, sharded=sharded, deferred=deferred, early=deferred)
    losses = []
    for _ in range(steps):
        losses.append(float(trainer.step().value.numpy()))
    dev.synchronize()
    np.savez(os.path.join(out_dir, f"rank{rank}_{mode}.npz"), *trainer.parameters_numpy(), losses=np.array(losses))
    dev.commDestroy()
    dev.close()


if __name__ == "__main__":
    main()
