"""Child process of tests/test_gpu_gemm_variants.py: matmul parity for a few shapes under whatever AIXB200_GEMM_* switches
the parent put in the environment (they are read once per process). Prints one JSON line."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from aix_b200 import BF16, F32, DeviceB200, TensorValue, from_storage, to_storage   # noqa: E402


def main():
    dev = DeviceB200(0)
    rng = np.random.default_rng(5)
    worst = {"bf16": 0.0, "f32": 0.0}
    repeatable = True
    shapes = [(256, 512, 512), (300, 200, 520), (1024, 1024, 1024), (2304, 640, 1792), (520, 1100, 264)]
    for dtype, name in ((BF16, "bf16"), (F32, "f32")):
        for m, k, n in shapes:
            a = from_storage(to_storage(rng.normal(0, 0.5, (m, k)).astype(np.float32), dtype), dtype).astype(np.float32)
            b = from_storage(to_storage(rng.normal(0, 0.5, (k, n)).astype(np.float32), dtype), dtype).astype(np.float32)
            want = a.astype(np.float64) @ b.astype(np.float64)
            for ta, tb in ((False, False), (True, False), (False, True)):
                A = TensorValue.from_numpy(a.T.copy() if ta else a, dev, dtype)
                B = TensorValue.from_numpy(b.T.copy() if tb else b, dev, dtype)
                if ta: A = A.transpose(0, 1)
                if tb: B = B.transpose(0, 1)
                got = A.matmul(B).numpy().astype(np.float64)
                again = A.matmul(B).numpy().astype(np.float64)
                repeatable = repeatable and bool(np.array_equal(got, again))
                worst[name] = max(worst[name], float(np.max(np.abs(got - want)) / np.max(np.abs(want))))
    dev.synchronize()
    print(json.dumps({"worst": worst, "repeatable": repeatable}))
    dev.close()


if __name__ == "__main__":
    main()
