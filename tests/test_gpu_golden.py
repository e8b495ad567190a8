"""The B200 device replays every golden case (tests/golden/make_golden.py) and must agree with the vectors the
reference's CPU device produced: integer results bit for bit, floats within the stated tolerance. This test needs
neither the reference sources nor the compiled reference library."""
import numpy as np
import pytest

from aix_b200 import BF16, DTYPE_NAMES, F16, F32, F64, TensorValue, from_storage
from test_oracle import GOLDEN, NAME_TO_DTYPE, load_cases

pytestmark = pytest.mark.gpu
FLOAT_TOL = {F64: 1e-12, F32: 1e-5, F16: 1e-2, BF16: 1e-2}


def test_device_reproduces_golden_vectors_of_the_reference(b200):
    golden = np.load(GOLDEN)
    produced = {}
    load_cases()(b200, lambda k, v: produced.__setitem__(k, np.array(v)))
    failures = []
    for key, got in produced.items():
        want = golden[key]
        parts = key.split("/")
        dtype = next((NAME_TO_DTYPE[p] for p in reversed(parts) if p in NAME_TO_DTYPE), F32)
        if parts[0] == "convert" and parts[2] in NAME_TO_DTYPE:
            dtype = NAME_TO_DTYPE[parts[2]]
        if got.shape != want.shape:
            failures.append(f"{key}: shape {got.shape} vs {want.shape}")
            continue
        if dtype not in FLOAT_TOL:
            if not np.array_equal(got, want):
                failures.append(f"{key}: integers differ {got.reshape(-1)[:6]} vs {want.reshape(-1)[:6]}")
            continue
        g = from_storage(got, dtype).astype(np.float64)
        w = from_storage(want, dtype).astype(np.float64)
        tol = FLOAT_TOL[dtype]
        scale = np.maximum(1.0, np.abs(w))
        if parts[0] == "reduce" and "sum" in parts[-1]:
            # the reference accumulates in the storage type; for 16-bit floats this device accumulates in f32
            x = from_storage(golden[f"reduce/{parts[1]}/x"], dtype).astype(np.float64)
            scale = np.maximum(1.0, np.abs(x).sum())
        if parts[0] == "matmul" and dtype in (F16, BF16):
            scale = np.maximum(1.0, np.abs(w).max()) * 4
        with np.errstate(invalid="ignore"):
            ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= tol * scale)
        if not ok.all():
            failures.append(f"{key}: {g[~ok][:3]} vs {w[~ok][:3]}")
    assert not failures, "\n".join(failures[:20])
    assert len(produced) > 500
