"""The C-ABI library loads without a GPU and exports every symbol include/aixb200.h declares; entry points validate
their arguments and report errors through status codes. No GPU is touched."""
import ctypes
import os
import re

import numpy as np
import pytest

from aix_b200 import _capi as C
from aix_b200 import DeviceB200, DeviceTensorParams, F32, I32, TensorValue

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "aixb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aixb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.load()
    names = declared_symbols()
    assert len(names) >= 55
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/aixb200.h but not exported"
    assert set(C.SIGNATURES) == set(names), set(C.SIGNATURES) ^ set(names)


def test_struct_layouts_match_the_header():
    assert ctypes.sizeof(C.Tensor) == 8 + 8 + 8 + 4 + 4 + 8 * 8 + 8 * 8
    assert ctypes.sizeof(C.Stats) == 8 * 24
    cfg = C.Config()
    C.load().aixb200_default_config(ctypes.byref(cfg))
    assert cfg.flush_threshold == 200 and cfg.fusion == 1 and cfg.dry_run == 0


def test_no_gpu_means_failure_not_fallback():
    lib = C.load()
    if lib.aixb200_device_count() > 0:
        pytest.skip("a GPU is visible")
    with pytest.raises(RuntimeError, match="no CUDA device|no CPU fallback"):
        DeviceB200(0)


def test_contract_violations_raise_value_error(dry):
    a = TensorValue.empty((4, 4), dry)
    bad = DeviceTensorParams(a.storage.data, F32, 0, (4, 4), 15, (4, 1))       # size does not match shape
    with pytest.raises(ValueError):
        dry.add(bad, a.deviceParams(), a.deviceParams())
    b = TensorValue.empty((3, 4), dry)
    with pytest.raises(ValueError):
        dry.matmul(a.deviceParams(), b.deviceParams(), a.deviceParams())        # inner dimensions differ
    with pytest.raises(ValueError):
        dry.argmax(a.deviceParams(), TensorValue.empty((), dry, F32).deviceParams())   # result must be int32
    with pytest.raises(ValueError):
        dry.deallocate(12345)
    p = dry.allocate(64)
    dry.deallocate(p)
    with pytest.raises(ValueError):
        DeviceTensorParams(p, F32, 0, (1,) * 9, 1, (1,) * 9).to_c()


def test_exchange_entry_points_without_a_communicator(dry):
    """No communicator (and no GPU): the joins are no-ops, the collectives are refused with a message, nothing crashes."""
    x = TensorValue.full(1.0, (16,), dry)
    dry.commWait()
    dry.commWaitFor(x.storage.data, 64)
    dry.commWaitFor(0, 0)
    for call in (dry.allReduce, dry.allReduceAsync):
        with pytest.raises(Exception, match="comm_init"):
            call(x.storage.data, 16, F32, 1.0)
    with pytest.raises(Exception, match="GPU"):
        dry.commInit(0, 1, bytes(C.COMM_ID_BYTES))
    dry.synchronize()
