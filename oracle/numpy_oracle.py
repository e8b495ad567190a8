"""TEST INFRASTRUCTURE - a numpy restatement of the reference's CPU device for the hot path.

`DeviceNumpyOracle` has the aix::Device method names and follows the loops of Targets/AIXLib/aixDeviceCPU.cpp op by op
(each method cites the lines it restates). It is pinned against the reference itself: tests/test_oracle.py checks it
against golden vectors that tests/golden/make_golden.py produced by running the reference's own CPU device
(oracle/_ref), and, where that library is present, against the live library on random inputs. Integer and byte
results must be identical; floating transcendental results may differ from the reference's libm in the last place
(numpy evaluates them in float64 and rounds once), which the tests bound at 1e-6 relative.

Only tests/, __graft_entry__.smoke() and the benchmark's CPU-baseline leg may import this module.
"""
import ctypes

import numpy as np

from aix_b200 import _capi as C
from aix_b200.device import (NUMPY_STORAGE, DeviceTensorParams, bfloat16_bits_to_float32, float32_to_bfloat16_bits, to_storage)

_INT_INFO = {C.I64: np.iinfo(np.int64), C.I32: np.iinfo(np.int32), C.I16: np.iinfo(np.int16), C.I8: np.iinfo(np.int8),
             C.U8: np.iinfo(np.uint8)}
_FLOATS = (C.F64, C.F32, C.F16, C.BF16)


def _is_float(dt):
    return dt in _FLOATS


class DeviceNumpyOracle:
    """Host memory, immediate execution, one thread - like aix::DeviceCPU."""

    def __init__(self):
        self._blocks = {}
        self.dry_run = False

    def name(self): return "CPU (numpy restatement)"
    def type(self): return 0

    # ---- memory (aixDeviceCPU.cpp:718-731) -------------------------------------------------------------------
    def allocate(self, size, dtype=None):
        nbytes = max(1, size if dtype is None else size * C.DTYPE_SIZES[dtype])
        buf = (ctypes.c_uint8 * (nbytes + 16))()
        addr = ctypes.addressof(buf)
        self._blocks[addr] = buf
        return addr

    def deallocate(self, memory):
        self._blocks.pop(memory, None)

    def emptyCache(self): pass
    def synchronize(self): pass

    def download(self, src, dtype, count, offset=0):
        out = np.empty(count, dtype=NUMPY_STORAGE[dtype])
        ctypes.memmove(out.ctypes.data, src + offset * C.DTYPE_SIZES[dtype], out.nbytes)
        return out

    # ---- views ----------------------------------------------------------------------------------------------------
    @staticmethod
    def _raw(addr, dtype, count):
        buf = (ctypes.c_uint8 * (count * C.DTYPE_SIZES[dtype])).from_address(addr)
        return np.frombuffer(buf, dtype=NUMPY_STORAGE[dtype])

    def _read(self, p: DeviceTensorParams, count=None):
        """Logical elements 0..count-1 of the view as a flat storage-typed array: physicalIndex
        (aixDeviceCPU.cpp:670-682) applied to every flat index; a one-element view repeats (index mod shape)."""
        count = p.size if count is None else count
        idx = np.arange(count, dtype=np.int64)
        off = np.full(count, p.offset, dtype=np.int64)
        rem = idx
        for dim in range(len(p.shape) - 1, -1, -1):
            off += (rem % p.shape[dim]) * p.strides[dim]
            rem = rem // p.shape[dim]
        span = int(off.max()) + 1 if count else 0
        return self._raw(p.data, p.dtype, span)[off]

    def _write(self, p: DeviceTensorParams, values):
        """Results are written densely from the storage base, res[i] (e.g. aixDeviceCPU.cpp:36-40)."""
        self._raw(p.data, p.dtype, len(values))[:] = values

    # ---- element-type helpers ---------------------------------------------------------------------------------
    @staticmethod
    def _to_compute(raw, dtype):
        """f16/bf16 values enter arithmetic as float32 (aixFloat16.hpp:104-122, 698-716)."""
        if dtype == C.BF16: return bfloat16_bits_to_float32(raw)
        if dtype == C.F16: return raw.astype(np.float32)
        return raw

    @staticmethod
    def _from_compute(x, dtype):
        if dtype == C.BF16: return float32_to_bfloat16_bits(x.astype(np.float32))
        if dtype == C.F16: return x.astype(np.float32).astype(np.float16)
        return x.astype(NUMPY_STORAGE[dtype], copy=False)

    @staticmethod
    def _convert(wide, dtype):
        """convertGenericValue (aixDeviceCPU.cpp:96-117) from a float-like value: integers saturate, NaN -> 0;
        f16/bf16 go through float (their only constructor takes float)."""
        if _is_float(dtype):
            if dtype == C.F64: return np.asarray(wide, dtype=np.float64)
            f = np.asarray(wide).astype(np.float32)
            return DeviceNumpyOracle._from_compute(f, dtype)
        info = _INT_INFO[dtype]
        w = np.asarray(wide, dtype=np.longdouble)
        w = np.where(np.isnan(w), np.longdouble(0), w)
        w = np.clip(w, np.longdouble(info.min), np.longdouble(info.max))
        out = np.trunc(w)
        if dtype == C.I64:
            # exact conversion of +-2^63 boundaries
            res = np.empty(out.shape, dtype=np.int64)
            hi = out >= np.longdouble(2) ** 63
            res[hi] = info.max
            res[~hi] = out[~hi].astype(np.int64)
            return res
        return out.astype(np.int64).astype(NUMPY_STORAGE[dtype])

    def _binary(self, a, b, r, fn):
        x = self._to_compute(self._read(a, r.size), r.dtype)
        y = self._to_compute(self._read(b, r.size), r.dtype)
        with np.errstate(all="ignore"):
            self._write(r, self._from_compute(fn(x, y), r.dtype))

    # ---- arithmetic (aixDeviceCPU.cpp:28-94) ---------------------------------------------------------------------
    def add(self, a, b, r): self._binary(a, b, r, lambda x, y: x + y)
    def sub(self, a, b, r): self._binary(a, b, r, lambda x, y: x - y)
    def mul(self, a, b, r): self._binary(a, b, r, lambda x, y: x * y)

    def div(self, a, b, r):
        if _is_float(r.dtype):
            return self._binary(a, b, r, lambda x, y: x / y)

        def truncdiv(x, y):           # C++ integer division truncates toward zero
            if np.any(y == 0):
                raise ZeroDivisionError("integer division by zero (the reference raises SIGFPE)")
            xi, yi = x.astype(np.int64), y.astype(np.int64)
            q = np.abs(xi) // np.abs(yi)
            return np.where((xi < 0) != (yi < 0), -q, q)
        self._binary(a, b, r, truncdiv)

    def unary(self, a, r):
        x = self._to_compute(self._read(a, r.size), r.dtype)
        with np.errstate(all="ignore"):
            self._write(r, self._from_compute(-x if _is_float(r.dtype) else (0 - x), r.dtype))

    # ---- fills (aixDeviceCPU.cpp:119-138) ------------------------------------------------------------------------
    def fill(self, scalar, scalarDType, r):
        raw = to_storage(np.array([scalar]), scalarDType)
        value = self.convert_array(raw, scalarDType, r.dtype)[0]
        self._write(r, np.full(r.size, value, dtype=NUMPY_STORAGE[r.dtype]))

    def fillMin(self, r):
        lowest = {C.F64: np.finfo(np.float64).min, C.F32: np.finfo(np.float32).min, C.F16: np.float16(-65504.0)}
        if r.dtype == C.BF16: value = np.uint16(0xFF7F)
        elif r.dtype in lowest: value = lowest[r.dtype]
        else: value = _INT_INFO[r.dtype].min
        self._write(r, np.full(r.size, value, dtype=NUMPY_STORAGE[r.dtype]))

    def convert_array(self, raw, src, dst):
        """copyGeneric / fillGeneric conversion rule (aixDeviceCPU.cpp:96-128, 408-424)."""
        if src == dst:
            return raw.copy()
        if _is_float(src):
            x = self._to_compute(raw, src)
            if _is_float(dst):
                if dst == C.F64: return x.astype(np.float64)
                return self._from_compute(x.astype(np.float32), dst)
            return self._convert(x.astype(np.longdouble), dst)
        if _is_float(dst):
            if dst == C.F64: return raw.astype(np.float64)
            return self._from_compute(raw.astype(np.float32), dst)
        return raw.astype(NUMPY_STORAGE[dst])          # integer -> integer: two's complement truncation

    def copy(self, src, srcDType, dst, dstDType, size):
        if size == 0: return
        self._raw(dst, dstDType, size)[:] = self.convert_array(self._raw(src, srcDType, size), srcDType, dstDType)

    copyImmediate = copy

    def contiguous(self, s, d):          # aixDeviceCPU.cpp:427-440
        self._write(d, self._read(s, d.size))

    # ---- math (aixDeviceCPU.cpp:155-242) ---------------------------------------------------------------------------
    def _wide_math(self, a, r, fn):
        """sqrt / log / exp / pow: evaluated in long double, then convertGenericValue back."""
        x = self._to_compute(self._read(a, r.size), r.dtype).astype(np.longdouble)
        with np.errstate(all="ignore"):
            self._write(r, self._convert(fn(x), r.dtype))

    def sqrt(self, a, r): self._wide_math(a, r, np.sqrt)
    def log(self, a, r):  self._wide_math(a, r, np.log)
    def exp(self, a, r):  self._wide_math(a, r, np.exp)

    def pow(self, a, e, r):
        x = self._to_compute(self._read(a, r.size), r.dtype).astype(np.longdouble)
        y = self._to_compute(self._read(e, r.size), r.dtype).astype(np.longdouble)
        with np.errstate(all="ignore"):
            self._write(r, self._convert(np.power(x, y), r.dtype))

    def _plain_math(self, a, r, fn):
        """sin / cos / tanh: std::sin(T) - float for f32/f16/bf16, double otherwise, integers truncate the double."""
        x = self._to_compute(self._read(a, r.size), r.dtype)
        with np.errstate(all="ignore"):
            # libm's results are (almost always) the correctly rounded ones: evaluate one precision up and round once.
            if r.dtype in (C.F32, C.F16, C.BF16):
                y = fn(x.astype(np.float64)).astype(np.float32)
                self._write(r, self._from_compute(y, r.dtype))
            elif r.dtype == C.F64:
                self._write(r, fn(x.astype(np.longdouble)).astype(np.float64))
            else:
                y = fn(x.astype(np.longdouble)).astype(np.float64)
                self._write(r, np.trunc(y).astype(np.int64).astype(NUMPY_STORAGE[r.dtype]))

    def sin(self, a, r):  self._plain_math(a, r, np.sin)
    def cos(self, a, r):  self._plain_math(a, r, np.cos)
    def tanh(self, a, r): self._plain_math(a, r, np.tanh)

    # ---- reductions (aixDeviceCPU.cpp:140-152, 245-255, 443-467) -----------------------------------------------------
    def _sequential_sum(self, values, dtype):
        """T sum = 0; sum += x for every element in order, rounding (or wrapping) in T after every addition."""
        if dtype in (C.F64, C.F32, C.F16):
            return np.cumsum(values, dtype=values.dtype)[-1] if len(values) else values.dtype.type(0)
        if dtype == C.BF16:
            acc = np.float32(0)
            for v in bfloat16_bits_to_float32(values):
                acc = bfloat16_bits_to_float32(float32_to_bfloat16_bits(np.float32(acc + v)))
            return float32_to_bfloat16_bits(np.float32(acc))
        return np.sum(values, dtype=values.dtype)                  # integers wrap; order does not matter

    def sum(self, a, r):
        self._write(r, np.array([self._sequential_sum(self._read(a), r.dtype)], dtype=NUMPY_STORAGE[r.dtype]))

    def max(self, a, r):
        raw = self._read(a)
        if r.dtype == C.BF16:
            self._write(r, np.array([raw[np.argmax(bfloat16_bits_to_float32(raw))]], dtype=np.uint16))
        else:
            self._write(r, np.array([raw.max()], dtype=raw.dtype))

    @staticmethod
    def _translation_index(count, dst_shape, src_shape):
        """translationIndex (aixDeviceCPU.cpp:627-649) for all flat source indices at once."""
        idx = np.arange(count, dtype=np.int64)
        original = np.zeros(count, dtype=np.int64)
        target_stride, original_stride = 1, 1
        j = len(dst_shape) - 1
        for i in range(len(src_shape) - 1, -1, -1):
            dim_index = (idx // target_stride) % src_shape[i]
            if j >= 0 and dst_shape[j] == src_shape[i]:
                original += dim_index * original_stride
                original_stride *= dst_shape[j]
                j -= 1
            elif j >= 0 and dst_shape[j] == 1:
                original_stride *= dst_shape[j]
                j -= 1
            target_stride *= src_shape[i]
        return original

    def reduceTo(self, s, d):
        src = self._to_compute(self._read(s), s.dtype)
        where = self._translation_index(s.size, tuple(d.shape), tuple(s.shape))
        out = self._raw(d.data, d.dtype, d.size)
        if d.dtype == C.BF16:
            acc = bfloat16_bits_to_float32(out).copy()
            for i, v in zip(where, src):       # sequential, rounding to bf16 after every addition
                acc[i] = bfloat16_bits_to_float32(float32_to_bfloat16_bits(np.float32(acc[i] + v)))
            out[:] = float32_to_bfloat16_bits(acc)
        else:
            np.add.at(out, where, src.astype(out.dtype))            # unbuffered: same order as the reference loop

    def maxTo(self, s, d):
        raw = self._read(s)
        where = self._translation_index(s.size, tuple(d.shape), tuple(s.shape))
        out = self._raw(d.data, d.dtype, d.size)
        if d.dtype == C.BF16:
            vals = bfloat16_bits_to_float32(out).copy()
            np.maximum.at(vals, where, bfloat16_bits_to_float32(raw))
            out[:] = float32_to_bfloat16_bits(vals)
        else:
            np.maximum.at(out, where, raw)

    def argmax(self, a, r):               # first maximal index (aixDeviceCPU.cpp:258-272)
        raw = self._to_compute(self._read(a), a.dtype)
        self._write(r, np.array([np.argmax(raw)], dtype=np.int32))

    def argmaxIndices(self, a, r):
        raw = self._to_compute(self._read(a), a.dtype)
        out = np.zeros(a.size, dtype=np.int32)
        out[np.argmax(raw)] = 1
        self._write(r, out)

    # ---- matmul (aixDeviceCPU.cpp:355-388): T sum = 0; sum += a*b in k order, every step rounded in T ---------------
    def matmul(self, a, b, r):
        m, k, n = a.shape[0], a.shape[1], b.shape[1]
        x = self._to_compute(self._read(a), r.dtype).reshape(m, k)
        y = self._to_compute(self._read(b), r.dtype).reshape(k, n)
        if r.dtype in (C.F16, C.BF16):
            q = lambda v: self._to_compute(self._from_compute(v, r.dtype), r.dtype)
            acc = np.zeros((m, n), dtype=np.float32)
            for kk in range(k):
                acc = q(acc + q(x[:, kk, None] * y[None, kk, :]))
            self._write(r, self._from_compute(acc, r.dtype).reshape(-1))
            return
        acc = np.zeros((m, n), dtype=x.dtype)
        with np.errstate(all="ignore"):
            for kk in range(k):
                acc = acc + x[:, kk, None] * y[None, kk, :]
        self._write(r, acc.reshape(-1))

    def transpose(self, a, r, dim0, dim1):   # aixDeviceCPU.cpp:391-405
        src = self._raw(a.data, a.dtype, a.size)
        idx = np.arange(a.size, dtype=np.int64)
        coords, rem = [], idx
        for st in a.strides:
            coords.append(rem // st)
            rem = rem % st
        coords[dim0], coords[dim1] = coords[dim1], coords[dim0]
        dst_index = sum(c * st for c, st in zip(coords, r.strides))
        self._raw(r.data, r.dtype, a.size)[dst_index] = src


# ---- whole-path restatements used where oracle/_ref is absent ----------------------------------------------------------
def chain_f32(a, b, c):
    """The config-0 expression op by op in float32, as the reference's CPU device evaluates it; returns (z, sum) with
    the sum accumulated sequentially in float32 (aixDeviceCPU.cpp:140-152)."""
    a, b, c = (np.asarray(v, dtype=np.float32) for v in (a, b, c))
    f32 = np.float32

    def exp32(x):
        return np.exp(x.astype(np.longdouble)).astype(f32)
    one = f32(1)
    sig = one / (one + exp32(-a))
    z = (a * b + c) * sig - np.tanh(b.astype(np.float64)).astype(f32) / (one + exp32(-c))
    return z.astype(f32), float(np.cumsum(z.reshape(-1), dtype=f32)[-1])
