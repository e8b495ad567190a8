"""Host-side mirror of the reference's device interface for the B200 device.

`DeviceB200` has one method per virtual of aix::Device (Targets/AIXLib/aixDevice.hpp:30-84), with the reference's
names and argument order, and forwards each call to the C ABI in include/aixb200.h. Contract violations raise
ValueError (the reference throws std::invalid_argument), CUDA / NVRTC / allocation failures raise RuntimeError
(std::runtime_error). Nothing here computes: without the built library or without a GPU the calls fail.
"""
import ctypes
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

from . import _capi as C

# numpy storage type of each element type (bf16 has no numpy type: raw uint16 bit patterns).
NUMPY_STORAGE = [np.float64, np.float32, np.float16, np.uint16, np.int64, np.int32, np.int16, np.int8, np.uint8]


def float32_to_bfloat16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns, NaN kept NaN (aixFloat16.hpp:775-805)."""
    x = np.asarray(x, dtype=np.float32)
    bits = np.ascontiguousarray(x).reshape(x.shape).view(np.uint32)
    nan = (bits & 0x7F800000 == 0x7F800000) & (bits & 0x007FFFFF != 0)
    rounded = (bits + (0x7FFF + ((bits >> 16) & 1))) >> 16
    return np.where(nan, (bits >> 16) | 0x0040, rounded).astype(np.uint16)


def bfloat16_bits_to_float32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint16)
    return (np.ascontiguousarray(b).reshape(b.shape).astype(np.uint32) << 16).view(np.float32)


def to_storage(values: np.ndarray, dtype: int) -> np.ndarray:
    """Converts an array of ordinary numpy numbers into the storage representation of `dtype`."""
    if dtype == C.BF16:
        return float32_to_bfloat16_bits(np.asarray(values, dtype=np.float32))
    values = np.asarray(values)
    return np.ascontiguousarray(values, dtype=NUMPY_STORAGE[dtype]).reshape(values.shape)


def from_storage(raw: np.ndarray, dtype: int) -> np.ndarray:
    """Storage representation -> ordinary numpy numbers (bf16 -> float32)."""
    return bfloat16_bits_to_float32(raw) if dtype == C.BF16 else raw


@dataclass
class DeviceTensorParams:
    """Mirror of aix::DeviceTensorParams (aixCore.hpp:189-198). `data` is an integer address."""
    data: int
    dtype: int = C.F32
    offset: int = 0
    shape: Sequence[int] = field(default_factory=tuple)
    size: int = 0
    strides: Sequence[int] = field(default_factory=tuple)

    def to_c(self) -> C.Tensor:
        cached = self.__dict__.get("_c")
        if cached is not None:
            return cached
        t = C.Tensor()
        t.data = self.data
        t.offset = self.offset
        t.size = self.size
        t.dtype = self.dtype
        if len(self.shape) > C.MAX_RANK:
            raise ValueError("rank above AIXB200_MAX_RANK")
        t.rank = len(self.shape)
        for i, (s, st) in enumerate(zip(self.shape, self.strides)):
            t.shape[i] = s
            t.strides[i] = st
        self.__dict__["_c"] = t        # descriptors are immutable once built: convert once
        return t

    @property
    def isContiguous(self) -> bool:
        expected = 1
        for s, st in zip(reversed(self.shape), reversed(self.strides)):
            if st != expected:
                return False
            expected *= s
        return True


_FILL_SCALARS: dict = {}


class DeviceB200:
    """One B200 GPU behind the aix::Device interface."""

    def __init__(self, ordinal: int = 0, **config):
        self._lib = C.load()
        cfg = C.Config()
        self._lib.aixb200_default_config(ctypes.byref(cfg))
        cfg.ordinal = ordinal
        for k, v in config.items():
            if not hasattr(cfg, k):
                raise ValueError(f"unknown configuration field {k}")
            setattr(cfg, k, v)
        handle = ctypes.c_void_p()
        status = self._lib.aixb200_create_with_config(ctypes.byref(cfg), ctypes.byref(handle))
        if status != C.OK:
            msg = self._lib.aixb200_last_error(None).decode()
            raise (ValueError if status == C.ERR_INVALID else RuntimeError)(f"DeviceB200: {msg}")
        self._h = handle
        self.dry_run = bool(cfg.dry_run)

    # ---- plumbing -------------------------------------------------------------------------------------------
    def _check(self, status: int):
        if status == C.OK:
            return
        msg = self._lib.aixb200_last_error(self._h).decode()
        if status == C.ERR_TIMEOUT:
            raise TimeoutError(msg)
        raise (ValueError if status == C.ERR_INVALID else RuntimeError)(msg)

    @staticmethod
    def _t(p: DeviceTensorParams):
        ref = p.__dict__.get("_ref")
        if ref is None:
            ref = p.__dict__["_ref"] = ctypes.byref(p.to_c())      # descriptors are immutable: one reference object per descriptor
        return ref

    def close(self):
        if getattr(self, "_h", None):
            self._lib.aixb200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- aix::Device ---------------------------------------------------------------------------------------
    def type(self) -> int:
        return 2                    # outside the reference's enum {kCPU = 0, kGPU_METAL = 1}

    def name(self) -> str:
        return self._lib.aixb200_name(self._h).decode()

    @staticmethod
    def dataTypeSize(dtype: int) -> int:
        return C.DTYPE_SIZES[dtype]

    def allocate(self, size: int, dtype: int | None = None) -> int:
        out = ctypes.c_void_p()
        if dtype is None:
            self._check(self._lib.aixb200_allocate(self._h, size, ctypes.byref(out)))
        else:
            self._check(self._lib.aixb200_allocate_typed(self._h, size, dtype, ctypes.byref(out)))
        return out.value

    def deallocate(self, memory: int):
        self._check(self._lib.aixb200_deallocate(self._h, memory))

    def add(self, a1, a2, result):  self._check(self._lib.aixb200_add(self._h, self._t(a1), self._t(a2), self._t(result)))
    def sub(self, a1, a2, result):  self._check(self._lib.aixb200_sub(self._h, self._t(a1), self._t(a2), self._t(result)))
    def mul(self, a1, a2, result):  self._check(self._lib.aixb200_mul(self._h, self._t(a1), self._t(a2), self._t(result)))
    def div(self, a1, a2, result):  self._check(self._lib.aixb200_div(self._h, self._t(a1), self._t(a2), self._t(result)))
    def unary(self, a1, result):    self._check(self._lib.aixb200_unary(self._h, self._t(a1), self._t(result)))

    def fill(self, scalar, scalarDType: int, result):
        key = (scalar, scalarDType)
        held = _FILL_SCALARS.get(key)
        if held is None:                   # the same few constants recur every step: keep their one-element buffers
            raw = to_storage(np.array([scalar]), scalarDType)
            held = (raw, raw.ctypes.data)
            if len(_FILL_SCALARS) < 4096:
                _FILL_SCALARS[key] = held
        self._check(self._lib.aixb200_fill(self._h, held[1], scalarDType, self._t(result)))

    def fillMin(self, result):      self._check(self._lib.aixb200_fill_min(self._h, self._t(result)))
    def sum(self, a, result):       self._check(self._lib.aixb200_sum(self._h, self._t(a), self._t(result)))
    def sqrt(self, a, result):      self._check(self._lib.aixb200_sqrt(self._h, self._t(a), self._t(result)))
    def sin(self, a, result):       self._check(self._lib.aixb200_sin(self._h, self._t(a), self._t(result)))
    def cos(self, a, result):       self._check(self._lib.aixb200_cos(self._h, self._t(a), self._t(result)))
    def tanh(self, a, result):      self._check(self._lib.aixb200_tanh(self._h, self._t(a), self._t(result)))
    def log(self, a, result):       self._check(self._lib.aixb200_log(self._h, self._t(a), self._t(result)))
    def exp(self, a, result):       self._check(self._lib.aixb200_exp(self._h, self._t(a), self._t(result)))
    def pow(self, a, exp, result):  self._check(self._lib.aixb200_pow(self._h, self._t(a), self._t(exp), self._t(result)))
    def max(self, a, result):       self._check(self._lib.aixb200_max(self._h, self._t(a), self._t(result)))
    def argmax(self, a, result):    self._check(self._lib.aixb200_argmax(self._h, self._t(a), self._t(result)))
    def argmaxIndices(self, a, result): self._check(self._lib.aixb200_argmax_indices(self._h, self._t(a), self._t(result)))
    def matmul(self, a, b, result): self._check(self._lib.aixb200_matmul(self._h, self._t(a), self._t(b), self._t(result)))

    def transpose(self, a, result, dim0: int, dim1: int):
        self._check(self._lib.aixb200_transpose(self._h, self._t(a), self._t(result), dim0, dim1))

    def copy(self, src: int, srcDType: int, dst: int, dstDType: int, size: int):
        self._check(self._lib.aixb200_copy(self._h, src, srcDType, dst, dstDType, size))

    def copyImmediate(self, src: int, srcDType: int, dst: int, dstDType: int, size: int):
        self._check(self._lib.aixb200_copy_immediate(self._h, src, srcDType, dst, dstDType, size))

    def contiguous(self, src, dst):  self._check(self._lib.aixb200_contiguous(self._h, self._t(src), self._t(dst)))
    def reduceTo(self, src, dst):    self._check(self._lib.aixb200_reduce_to(self._h, self._t(src), self._t(dst)))
    def maxTo(self, src, dst):       self._check(self._lib.aixb200_max_to(self._h, self._t(src), self._t(dst)))
    def argmaxTo(self, src, dst, dim: int): self._check(self._lib.aixb200_argmax_to(self._h, self._t(src), self._t(dst), dim))
    def argmaxIndicesTo(self, src, dst, dim: int):
        self._check(self._lib.aixb200_argmax_indices_to(self._h, self._t(src), self._t(dst), dim))

    def sliceSet(self, src, dst, dim: int, start: int, end: int, step: int):
        self._check(self._lib.aixb200_slice_set(self._h, self._t(src), self._t(dst), dim, start, end, step))

    def tril(self, src, dst, diagonal: int): self._check(self._lib.aixb200_tril(self._h, self._t(src), self._t(dst), diagonal))
    def triu(self, src, dst, diagonal: int): self._check(self._lib.aixb200_triu(self._h, self._t(src), self._t(dst), diagonal))

    def indexSelect(self, src, dst, indices, dim: int):
        self._check(self._lib.aixb200_index_select(self._h, self._t(src), self._t(dst), self._t(indices), dim))

    def indexAdd(self, src, dst, indices, dim: int):
        self._check(self._lib.aixb200_index_add(self._h, self._t(src), self._t(dst), self._t(indices), dim))

    def emptyCache(self):   self._check(self._lib.aixb200_empty_cache(self._h))
    def synchronize(self):  self._check(self._lib.aixb200_synchronize(self._h))

    # ---- additions over the reference interface ----------------------------------------------------------------
    def sumStaticScratch(self, a, result):
        """Device::sum without any allocation on the way: partials go to a static device array of the library.
        For callers that cannot allocate when they call (fixed memory budget, allocation-free regions). Inputs must be
        device memory, at most 2**30 elements, and recorded work must have been synchronised before."""
        self._check(self._lib.aixb200_sum_static_scratch(self._h, self._t(a), self._t(result)))

    def stats(self) -> dict:
        s = C.Stats()
        self._check(self._lib.aixb200_get_stats(self._h, ctypes.byref(s)))
        return s.as_dict()

    def lastKernelSource(self) -> str | None:
        s = self._lib.aixb200_last_kernel_source(self._h)
        return s.decode() if s else None

    def flushL2(self):  self._check(self._lib.aixb200_flush_l2(self._h))

    def selfTestBoundedWait(self, limit_ns: int = 1_000_000):
        self._check(self._lib.aixb200_self_test_bounded_wait(self._h, limit_ns))

    def createEvent(self) -> int:
        ev = ctypes.c_void_p()
        self._check(self._lib.aixb200_event_create(self._h, ctypes.byref(ev)))
        return ev.value

    def recordEvent(self, ev: int):  self._check(self._lib.aixb200_event_record(self._h, ev))

    def elapsedMs(self, start: int, stop: int) -> float:
        ms = ctypes.c_float()
        self._check(self._lib.aixb200_event_elapsed_ms(self._h, start, stop, ctypes.byref(ms)))
        return ms.value

    def destroyEvent(self, ev: int): self._check(self._lib.aixb200_event_destroy(self._h, ev))

    @staticmethod
    def commUniqueId() -> bytes:
        buf = ctypes.create_string_buffer(C.COMM_ID_BYTES)
        if C.load().aixb200_comm_unique_id(buf) != C.OK:
            raise RuntimeError(C.load().aixb200_last_error(None).decode())
        return buf.raw

    def commInit(self, rank: int, nranks: int, unique_id: bytes):
        self._check(self._lib.aixb200_comm_init(self._h, rank, nranks, ctypes.c_char_p(unique_id)))

    def allReduce(self, data: int, count: int, dtype: int, scale: float = 1.0):
        self._check(self._lib.aixb200_all_reduce(self._h, data, count, dtype, scale))

    def allReduceAsync(self, data: int, count: int, dtype: int, scale: float = 1.0):
        self._check(self._lib.aixb200_all_reduce_async(self._h, data, count, dtype, scale))

    def reduceScatterAsync(self, data: int, count: int, dtype: int, scale: float = 1.0):
        self._check(self._lib.aixb200_reduce_scatter_async(self._h, data, count, dtype, scale))

    def allGatherAsync(self, data: int, count: int, dtype: int):
        self._check(self._lib.aixb200_all_gather_async(self._h, data, count, dtype))

    def commRank(self):
        rank, size = ctypes.c_int(), ctypes.c_int()
        self._check(self._lib.aixb200_comm_rank(self._h, ctypes.byref(rank), ctypes.byref(size)))
        return rank.value, size.value

    def commWait(self): self._check(self._lib.aixb200_comm_wait(self._h))

    def commWaitFor(self, data: int, nbytes: int): self._check(self._lib.aixb200_comm_wait_for(self._h, data, nbytes))

    def commDestroy(self): self._check(self._lib.aixb200_comm_destroy(self._h))

    # Host <-> device helpers built on copy / copyImmediate (what TensorValue's host-pointer constructor and
    # host reads do in the reference, aixCore.hpp:249-259, 435-440).
    def upload(self, host: np.ndarray, dtype: int, dst: int | None = None) -> int:
        raw = np.ascontiguousarray(host)
        assert raw.dtype == NUMPY_STORAGE[dtype], "pass storage-typed data (see to_storage)"
        if dst is None:
            dst = self.allocate(raw.size, dtype)
        self.copy(raw.ctypes.data, dtype, dst, dtype, raw.size)
        self._keepalive = raw
        return dst

    def download(self, src: int, dtype: int, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=NUMPY_STORAGE[dtype])
        if self.dry_run:
            self.synchronize()
            ctypes.memmove(out.ctypes.data, src + offset * C.DTYPE_SIZES[dtype], out.nbytes)
            return out
        self.copyImmediate(src + offset * C.DTYPE_SIZES[dtype], dtype, out.ctypes.data, dtype, count)
        return out
