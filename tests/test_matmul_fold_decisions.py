"""Which recorded consumers an f32 matmul takes into its epilogue - the host-side decision, on a dry-run device (nothing is
launched; the device counts what it would have folded). nn::Linear is matmul(x, W) + b followed by tanh
(aixNeuralNetwork.hpp:150-153): the add and the tanh are folded as far as the values they consume are dead, so that the
product's kernel is left with one output; values that stay alive keep their own kernels."""
import os

import numpy as np
import pytest

from aix_b200 import F32, DeviceB200, TensorValue


@pytest.fixture(scope="module")
def deep():
    """A dry-run device that folds the tanh as well (AIXB200_GEMM_EPILOGUE=2, read when a device is created; the default
    folds the add only)."""
    old = os.environ.get("AIXB200_GEMM_EPILOGUE")
    os.environ["AIXB200_GEMM_EPILOGUE"] = "2"
    try:
        dev = DeviceB200(0, dry_run=1, disk_cache=0)
    finally:
        if old is None: os.environ.pop("AIXB200_GEMM_EPILOGUE")
        else: os.environ["AIXB200_GEMM_EPILOGUE"] = old
    yield dev
    dev.close()


def run(dry, body):
    dry.synchronize()
    before = dry.stats()
    kept = body()
    dry.synchronize()
    after = dry.stats()
    del kept
    return {k: after[k] - before[k] for k in ("matmul_consumers_folded", "fused_kernels", "ops_recorded")}


def operands(dry, m=256, k=128, n=256):
    x, w = TensorValue.full(0.5, (m, k), dry), TensorValue.full(0.25, (k, n), dry)
    b = TensorValue.full(0.1, (1, n), dry)
    return x, w, b


def test_by_default_the_add_is_folded_when_no_recorded_op_consumes_the_sum(dry):
    x, w, b = operands(dry)
    d = run(dry, lambda: (x.matmul(w) + b).tanh())
    assert d["matmul_consumers_folded"] == 0 and d["fused_kernels"] == 1, d        # the product, then add + tanh as one kernel
    d = run(dry, lambda: x.matmul(w) + b)
    assert d["matmul_consumers_folded"] == 1 and d["fused_kernels"] == 0, d        # nothing recorded consumes the sum
    d = run(dry, lambda: (x.matmul(w) + b).matmul(w.transpose(0, 1)))
    assert d["matmul_consumers_folded"] == 1 and d["fused_kernels"] == 0, d        # straight into the next product


def test_dead_intermediates_are_folded_and_live_ones_are_not(deep):
    dry = deep
    x, w, b = operands(dry)
    d = run(dry, lambda: (x.matmul(w) + b).tanh())
    assert d["matmul_consumers_folded"] == 2 and d["fused_kernels"] == 0, d        # one product, nothing else

    def all_alive():
        mm = x.matmul(w)
        s = mm + b
        return mm, s, s.tanh()
    d = run(dry, all_alive)
    assert d["matmul_consumers_folded"] == 0 and d["fused_kernels"] == 1, d        # add + tanh as one generated kernel

    def sum_alive():
        s = x.matmul(w) + b
        return s, s.tanh()
    d = run(dry, sum_alive)
    assert d["matmul_consumers_folded"] == 1 and d["fused_kernels"] == 1, d        # the tanh keeps its kernel


def test_what_does_not_match_is_left_alone(deep):
    dry = deep
    x, w, b = operands(dry)
    full = TensorValue.full(0.1, (256, 256), dry)
    column = TensorValue.full(0.1, (256, 1), dry)
    assert run(dry, lambda: x.matmul(w) + full)["matmul_consumers_folded"] == 0
    assert run(dry, lambda: x.matmul(w) + column)["matmul_consumers_folded"] == 0
    assert run(dry, lambda: x.matmul(w) * b)["matmul_consumers_folded"] == 0
    assert run(dry, lambda: (x.matmul(w) + b).exp())["matmul_consumers_folded"] == 1          # the add alone
    assert run(dry, lambda: b + x.matmul(w))["matmul_consumers_folded"] == 1                  # row vector on the left
    # shapes the folding kernel does not take: at most 128 rows, a row length that is no multiple of four
    xs, ws, bs = operands(dry, 128, 128, 256)
    assert run(dry, lambda: (xs.matmul(ws) + bs).tanh())["matmul_consumers_folded"] == 0
    xo, wo, bo = operands(dry, 256, 128, 250)
    assert run(dry, lambda: (xo.matmul(wo) + bo).tanh())["matmul_consumers_folded"] == 0

    def product_read_again():
        mm = x.matmul(w)
        s = mm + b
        e = mm * 0.5
        del mm
        t = s.tanh()
        del s
        return e, t
    assert run(dry, product_read_again)["matmul_consumers_folded"] == 0


def test_ops_recorded_while_the_product_waits_do_not_end_the_wait(deep):
    dry = deep
    x, w, b = operands(dry)

    def with_bystanders():
        s = x.matmul(w) + b
        other = TensorValue.full(3.0, (1000,), dry)       # touches nothing of the product
        b2 = b * 2.0                                       # reads the bias, writes elsewhere
        t = s.tanh()
        del s
        return other, b2, t
    d = run(dry, with_bystanders)
    assert d["matmul_consumers_folded"] == 2, d


def test_strict_math_and_the_switch_keep_every_product_in_its_own_call():
    from aix_b200 import DeviceB200
    strict = DeviceB200(0, dry_run=1, disk_cache=0, strict_math=1)
    try:
        x, w, b = operands(strict)
        assert run(strict, lambda: (x.matmul(w) + b).tanh())["matmul_consumers_folded"] == 0
        del x, w, b
    finally:
        strict.close()


def test_a_dead_product_is_written_straight_into_a_zero_filled_accumulation_target(dry):
    """zeroGrad() fills every gradient, backward() then does `grad += x^T . G` (aixCore.hpp:2014-2021, 2192-2207): the zero-fill is
    still recorded and the product is a temporary, so the product lands in the gradient buffer and neither the fill nor the
    add runs."""
    x, w, b = operands(dry)

    def accumulate():
        g = TensorValue.full(0.0, (256, 256), dry)
        g += x.matmul(w)
        return g
    d = run(dry, accumulate)
    assert d["matmul_consumers_folded"] == 1 and d["fused_kernels"] == 0, d

    def product_kept():
        g = TensorValue.full(0.0, (256, 256), dry)
        mm = x.matmul(w)
        g += mm
        return g, mm
    d = run(dry, product_kept)
    assert d["matmul_consumers_folded"] == 0 and d["fused_kernels"] == 1, d

    def target_not_zero():
        g = TensorValue.full(1.0, (256, 256), dry)
        g += x.matmul(w)
        return g
    d = run(dry, target_not_zero)
    assert d["matmul_consumers_folded"] == 0 and d["fused_kernels"] == 1, d

    def target_read_in_between():
        g = TensorValue.full(0.0, (256, 256), dry)
        h = g * 2.0
        g += x.matmul(w)
        return g, h
    d = run(dry, target_read_in_between)
    assert d["matmul_consumers_folded"] == 0, d
