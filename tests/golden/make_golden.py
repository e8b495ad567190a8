"""Generates tests/golden/golden_ops.npz by running the reference's own CPU device (oracle/_ref/libaixref.so, built from
the reference sources by oracle/build_ref.py) on small seeded inputs. The file pins the numpy oracle and the GPU path
to the reference on machines where the reference library is not available.

    python tests/golden/make_golden.py

Every array is stored in its storage representation (bf16 as uint16 bit patterns).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from aix_b200 import BF16, DTYPE_NAMES, F16, F32, F64, I8, I16, I32, I64, U8, TensorValue, scalar_like, to_storage  # noqa: E402

ALL = [F64, F32, F16, BF16, I64, I32, I16, I8, U8]
FLOATS = [F64, F32, F16, BF16]
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_ops.npz")


def inputs(rng, n, dtype, positive=False, small=False):
    if dtype in FLOATS:
        return rng.uniform(0.1 if positive else -2.0, 2.0, n)
    if dtype == U8:
        return rng.integers(1 if positive else 0, 12 if small else 200, n)
    return rng.integers(1 if positive else (-6 if small else -90), 7 if small else 90, n)


def cases(dev, store):
    """Runs every case on `dev`; `store(name, array)` receives inputs and outputs. Inputs are recorded too, so that a
    consumer can replay the case on another device without re-deriving the random stream."""
    rng = np.random.default_rng(20240101)
    n = 41
    for dt in ALL:
        name = DTYPE_NAMES[dt]
        for op in ("add", "sub", "mul", "div", "pow"):
            small = op in ("mul", "pow")
            x = inputs(rng, n, dt, positive=(op == "pow"), small=small)
            y = inputs(rng, n, dt, positive=(op in ("div", "pow")), small=small)
            if op == "pow" and dt not in FLOATS:
                y = np.minimum(y, 3)
            a, b = TensorValue.from_numpy(x, dev, dt), TensorValue.from_numpy(y, dev, dt)
            r = {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "div": lambda: a / b, "pow": lambda: a.pow(b)}[op]()
            store(f"binary/{op}/{name}/x", a.raw()); store(f"binary/{op}/{name}/y", b.raw()); store(f"binary/{op}/{name}/out", r.raw())
        for op in ("unary", "sqrt", "sin", "cos", "tanh", "log", "exp"):
            x = inputs(rng, n, dt, positive=(op in ("sqrt", "log")), small=(op == "exp"))
            a = TensorValue.from_numpy(x, dev, dt)
            r = TensorValue.empty(a.shape, dev, dt)
            getattr(dev, op)(a.deviceParams(), r.deviceParams())          # the device call itself, also on integer tensors
            store(f"unary/{op}/{name}/x", a.raw()); store(f"unary/{op}/{name}/out", r.raw())
        for value in (3.7, -3.7, 1e10, -1e10, 300.0, -300.0, 0.0):
            store(f"fill/{name}/{value}", TensorValue.full(value, (5,), dev, dt).raw())
        t = TensorValue.empty((5,), dev, dt)
        dev.fillMin(t.deviceParams())
        store(f"fillmin/{name}", t.raw())
        x = rng.uniform(-300, 300, 33)
        src = TensorValue.from_numpy(np.clip(x, 0, 200) if dt == U8 else x, dev, dt)
        store(f"convert/{name}/x", src.raw())
        for dst in ALL:
            store(f"convert/{name}/{DTYPE_NAMES[dst]}", src.to(dst).raw())
        # reductions
        x = inputs(rng, 6 * 7, dt).reshape(6, 7)
        t = TensorValue.from_numpy(x, dev, dt)
        store(f"reduce/{name}/x", t.raw())
        store(f"reduce/{name}/sum", t.sum().raw()); store(f"reduce/{name}/max", t.max().raw())
        store(f"reduce/{name}/sum0", t.sum(0).raw()); store(f"reduce/{name}/sum1", t.sum(1).raw())
        store(f"reduce/{name}/max0", t.max(0).raw()); store(f"reduce/{name}/max1", t.max(1).raw())
        store(f"reduce/{name}/sumT", t.transpose(0, 1).sum().raw())
        # matmul with plain and transposed operands
        a = inputs(rng, 5 * 4, dt, small=True).reshape(5, 4)
        b = inputs(rng, 4 * 3, dt, small=True).reshape(4, 3)
        ta, tb = TensorValue.from_numpy(a, dev, dt), TensorValue.from_numpy(b, dev, dt)
        store(f"matmul/{name}/a", ta.raw()); store(f"matmul/{name}/b", tb.raw())
        store(f"matmul/{name}/ab", ta.matmul(tb).raw())
        store(f"matmul/{name}/atbt", tb.transpose(0, 1).matmul(ta.transpose(0, 1)).raw())
    # broadcast + in-place + scalars, f32 and bf16
    for dt in (F32, BF16):
        name = DTYPE_NAMES[dt]
        x = rng.uniform(-1, 1, (9, 12)); row = rng.uniform(0.5, 1.5, 12); col = rng.uniform(-1, 1, (9, 1))
        tx, tr, tc = (TensorValue.from_numpy(v, dev, dt) for v in (x, row, col))
        y = tx * tr + tc
        y = y - tx.transpose(0, 1).contiguous().transpose(0, 1) + scalar_like(3.0, y)
        m = TensorValue.from_numpy(x, dev, dt)
        m *= 0.9
        m += 0.1 * y
        store(f"broadcast/{name}/x", tx.raw()); store(f"broadcast/{name}/row", tr.raw()); store(f"broadcast/{name}/col", tc.raw())
        store(f"broadcast/{name}/y", y.raw()); store(f"broadcast/{name}/m", m.raw())
    # config-0 expression through the reference's aix::Tensor front end
    a, b, c = (np.random.default_rng(0).uniform(-1, 1, (3, 64, 64)).astype(np.float32))
    if hasattr(dev, "chain_f32"):
        z, s, _ = dev.chain_f32(a, b, c)
        store("chain/a", a); store("chain/b", b); store("chain/c", c); store("chain/z", z); store("chain/sum", np.array([s], dtype=np.float32))
    # MLP training through the reference's nn / optim classes: 3 Adam steps on a tiny tanh MLP
    if hasattr(dev, "mlp_train_f32"):
        g = np.random.default_rng(7)
        dims = [6, 10, 8, 4]
        ws = [g.uniform(-0.5, 0.5, (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
        bs = [g.uniform(-0.5, 0.5, (1, dims[i + 1])).astype(np.float32) for i in range(3)]
        x = g.normal(0, 1, (5, 6)).astype(np.float32); y = g.normal(0, 1, (5, 4)).astype(np.float32)
        for i in range(3):
            store(f"mlp/w{i}_init", ws[i].copy()); store(f"mlp/b{i}_init", bs[i].copy())
        losses, _ = dev.mlp_train_f32(dims, ws, bs, x, y, steps=3, lr=1e-3)
        store("mlp/x", x); store("mlp/y", y); store("mlp/losses", losses)
        for i in range(3):
            store(f"mlp/w{i}_final", ws[i]); store(f"mlp/b{i}_final", bs[i])


if __name__ == "__main__":
    from oracle.ref_device import DeviceRefCPU
    data = {}
    cases(DeviceRefCPU(), lambda k, v: data.__setitem__(k, np.array(v)))
    np.savez_compressed(OUT, **data)
    print(f"{len(data)} arrays, {os.path.getsize(OUT)} bytes -> {OUT}")
