"""Pins the numpy oracle to the reference: (a) against the committed golden vectors that the reference's own CPU
device produced (tests/golden/make_golden.py), (b) where oracle/_ref is present, against the live reference library.
Integer, byte, arithmetic, conversion, reduction and matmul results must be bit-identical; transcendental results
may differ in the last place (float64 evaluation in numpy vs the reference's libm)."""
import importlib.util
import os

import numpy as np
import pytest

from aix_b200 import BF16, DTYPE_NAMES, F16, F32, F64, from_storage
from oracle.numpy_oracle import DeviceNumpyOracle, chain_f32

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "golden_ops.npz")
NAME_TO_DTYPE = {n: i for i, n in enumerate(DTYPE_NAMES)}
TRANSCENDENTAL = ("sqrt", "sin", "cos", "tanh", "log", "exp", "pow")


def load_cases():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.cases


def compare(key, got, want):
    parts = key.split("/")
    dtype = next((NAME_TO_DTYPE[p] for p in reversed(parts) if p in NAME_TO_DTYPE), F32)
    if parts[0] == "convert":
        dtype = NAME_TO_DTYPE[parts[2]] if parts[2] in NAME_TO_DTYPE else NAME_TO_DTYPE[parts[1]]
    assert got.shape == want.shape, key
    inexact = len(parts) > 1 and parts[1] in TRANSCENDENTAL and dtype in (F64, F32, F16, BF16)
    if not inexact:
        assert np.array_equal(got, want, equal_nan=(got.dtype.kind == "f")), f"{key}: oracle differs from the reference"
        return
    g = from_storage(got, dtype).astype(np.float64)
    w = from_storage(want, dtype).astype(np.float64)
    tol = {F64: 1e-13, F32: 1e-6, F16: 2.0 ** -10, BF16: 2.0 ** -7}[dtype]
    with np.errstate(invalid="ignore"):
        ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= tol * np.abs(w))
    assert ok.all(), f"{key}: {g[~ok][:3]} vs {w[~ok][:3]}"


def test_oracle_reproduces_golden_vectors_of_the_reference():
    golden = np.load(GOLDEN)
    produced = {}
    load_cases()(DeviceNumpyOracle(), lambda k, v: produced.__setitem__(k, np.array(v)))
    checked = 0
    for key, value in produced.items():
        assert key in golden.files, key
        compare(key, value, golden[key])
        checked += 1
    assert checked > 500


def test_chain_restatement_matches_golden_front_end_run():
    golden = np.load(GOLDEN)
    z, s = chain_f32(golden["chain/a"], golden["chain/b"], golden["chain/c"])
    assert np.allclose(z, golden["chain/z"], rtol=1e-6, atol=1e-7)
    assert abs(s - float(golden["chain/sum"][0])) <= 1e-5 * np.abs(golden["chain/z"]).sum()


def test_oracle_matches_live_reference_on_random_inputs(ref):
    """Only where oracle/_ref is built: a second seed, larger arrays, same comparison rules."""
    from aix_b200 import TensorValue
    rng = np.random.default_rng(99)
    oracle = DeviceNumpyOracle()
    for dt in range(9):
        x = rng.integers(1, 50, 300) if dt > BF16 else rng.uniform(0.2, 3.0, 300)
        y = rng.integers(1, 9, 300) if dt > BF16 else rng.uniform(0.2, 3.0, 300)
        outs = []
        for dev in (oracle, ref):
            a, b = TensorValue.from_numpy(x, dev, dt), TensorValue.from_numpy(y, dev, dt)
            r = ((a * b + a) / b - a)
            outs.append((r.raw(), r.sum().raw(), r.max().raw(), r.reshape((20, 15)).sum(0).raw(), r.reshape((20, 15)).max(1).raw()))
        for g, w in zip(*outs):
            assert np.array_equal(g, w), DTYPE_NAMES[dt]
