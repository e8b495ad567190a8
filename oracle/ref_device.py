"""TEST INFRASTRUCTURE - the reference's own CPU device (aix::DeviceCPU) behind the aix::Device method names.

Loads oracle/_ref/libaixref.so (built by oracle/build_ref.py from the reference sources) and exposes the same Python
interface as aix_b200.DeviceB200, so one test body can drive both. Only tests, the smoke check and the benchmark's
CPU-baseline leg may import this module; nothing in the product does.
"""
import ctypes
import os

import numpy as np

from aix_b200 import _capi as C
from aix_b200.device import NUMPY_STORAGE, DeviceTensorParams, to_storage

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libaixref.so")
_T = ctypes.POINTER(C.Tensor)


def available() -> bool:
    return os.path.isfile(LIB_PATH)


class DeviceRefCPU:
    def __init__(self):
        if not available():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python oracle/build_ref.py` where the reference sources are")
        lib = ctypes.CDLL(LIB_PATH)
        lib.aixref_allocate.restype = ctypes.c_void_p
        lib.aixref_allocate.argtypes = [ctypes.c_size_t]
        lib.aixref_deallocate.argtypes = [ctypes.c_void_p]
        for n in ("add", "sub", "mul", "div", "pow", "matmul"):
            getattr(lib, "aixref_" + n).argtypes = [_T, _T, _T]
        for n in ("unary", "sqrt", "sin", "cos", "tanh", "log", "exp", "sum", "max", "argmax", "argmax_indices",
                  "contiguous", "reduce_to", "max_to"):
            getattr(lib, "aixref_" + n).argtypes = [_T, _T]
        lib.aixref_fill.argtypes = [ctypes.c_void_p, ctypes.c_uint32, _T]
        lib.aixref_fill_min.argtypes = [_T]
        lib.aixref_copy.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_size_t]
        lib.aixref_transpose.argtypes = [_T, _T, ctypes.c_size_t, ctypes.c_size_t]
        lib.aixref_argmax_to.argtypes = [_T, _T, ctypes.c_size_t]
        lib.aixref_argmax_indices_to.argtypes = [_T, _T, ctypes.c_size_t]
        lib.aixref_slice_set.argtypes = [_T, _T] + [ctypes.c_size_t] * 4
        lib.aixref_tril.argtypes = [_T, _T, ctypes.c_int64]
        lib.aixref_triu.argtypes = [_T, _T, ctypes.c_int64]
        lib.aixref_index_select.argtypes = [_T, _T, _T, ctypes.c_size_t]
        lib.aixref_index_add.argtypes = [_T, _T, _T, ctypes.c_size_t]
        lib.aixref_chain_f32.restype = ctypes.c_double
        lib.aixref_chain_f32.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 2 + [ctypes.c_void_p] * 2
        lib.aixref_mlp_train_f32.restype = ctypes.c_double
        lib.aixref_mlp_train_f32.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p]
        self._lib = lib
        self.dry_run = False

    @staticmethod
    def _t(p: DeviceTensorParams):
        return ctypes.byref(p.to_c())

    def name(self): return "CPU"
    def type(self): return 0

    def allocate(self, size, dtype=None):
        nbytes = size if dtype is None else size * C.DTYPE_SIZES[dtype]
        return self._lib.aixref_allocate(max(nbytes, 1))

    def deallocate(self, memory): self._lib.aixref_deallocate(memory)

    def add(self, a, b, r): self._lib.aixref_add(self._t(a), self._t(b), self._t(r))
    def sub(self, a, b, r): self._lib.aixref_sub(self._t(a), self._t(b), self._t(r))
    def mul(self, a, b, r): self._lib.aixref_mul(self._t(a), self._t(b), self._t(r))
    def div(self, a, b, r): self._lib.aixref_div(self._t(a), self._t(b), self._t(r))
    def pow(self, a, b, r): self._lib.aixref_pow(self._t(a), self._t(b), self._t(r))
    def matmul(self, a, b, r): self._lib.aixref_matmul(self._t(a), self._t(b), self._t(r))
    def unary(self, a, r): self._lib.aixref_unary(self._t(a), self._t(r))
    def sqrt(self, a, r): self._lib.aixref_sqrt(self._t(a), self._t(r))
    def sin(self, a, r): self._lib.aixref_sin(self._t(a), self._t(r))
    def cos(self, a, r): self._lib.aixref_cos(self._t(a), self._t(r))
    def tanh(self, a, r): self._lib.aixref_tanh(self._t(a), self._t(r))
    def log(self, a, r): self._lib.aixref_log(self._t(a), self._t(r))
    def exp(self, a, r): self._lib.aixref_exp(self._t(a), self._t(r))
    def sum(self, a, r): self._lib.aixref_sum(self._t(a), self._t(r))
    def max(self, a, r): self._lib.aixref_max(self._t(a), self._t(r))
    def argmax(self, a, r): self._lib.aixref_argmax(self._t(a), self._t(r))
    def argmaxIndices(self, a, r): self._lib.aixref_argmax_indices(self._t(a), self._t(r))
    def contiguous(self, s, d): self._lib.aixref_contiguous(self._t(s), self._t(d))
    def reduceTo(self, s, d): self._lib.aixref_reduce_to(self._t(s), self._t(d))
    def maxTo(self, s, d): self._lib.aixref_max_to(self._t(s), self._t(d))

    def fill(self, scalar, scalarDType, result):
        raw = to_storage(np.array([scalar]), scalarDType)
        self._lib.aixref_fill(raw.ctypes.data, scalarDType, self._t(result))

    def fillMin(self, result): self._lib.aixref_fill_min(self._t(result))
    def copy(self, src, sdt, dst, ddt, n): self._lib.aixref_copy(src, sdt, dst, ddt, n)
    def copyImmediate(self, src, sdt, dst, ddt, n): self._lib.aixref_copy(src, sdt, dst, ddt, n)
    def transpose(self, a, r, d0, d1): self._lib.aixref_transpose(self._t(a), self._t(r), d0, d1)
    def argmaxTo(self, s, d, dim): self._lib.aixref_argmax_to(self._t(s), self._t(d), dim)
    def argmaxIndicesTo(self, s, d, dim): self._lib.aixref_argmax_indices_to(self._t(s), self._t(d), dim)
    def sliceSet(self, s, d, dim, start, end, step): self._lib.aixref_slice_set(self._t(s), self._t(d), dim, start, end, step)
    def tril(self, s, d, diagonal): self._lib.aixref_tril(self._t(s), self._t(d), diagonal)
    def triu(self, s, d, diagonal): self._lib.aixref_triu(self._t(s), self._t(d), diagonal)
    def indexSelect(self, s, d, idx, dim): self._lib.aixref_index_select(self._t(s), self._t(d), self._t(idx), dim)
    def indexAdd(self, s, d, idx, dim): self._lib.aixref_index_add(self._t(s), self._t(d), self._t(idx), dim)
    def emptyCache(self): pass
    def synchronize(self): pass

    def download(self, src, dtype, count, offset=0):
        out = np.empty(count, dtype=NUMPY_STORAGE[dtype])
        ctypes.memmove(out.ctypes.data, src + offset * C.DTYPE_SIZES[dtype], out.nbytes)
        return out

    # ---- whole-path drivers through the reference's front end (oracle/ref_shim.cpp) ------------------------------
    def chain_f32(self, a, b, c):
        """z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c)) and z.sum() through aix::Tensor on the CPU device.
        Returns (z, sum, seconds)."""
        a, b, c = (np.ascontiguousarray(x, dtype=np.float32) for x in (a, b, c))
        rows, cols = a.shape
        z = np.empty_like(a)
        s = ctypes.c_float()
        secs = self._lib.aixref_chain_f32(a.ctypes.data, b.ctypes.data, c.ctypes.data, rows, cols, z.ctypes.data, ctypes.byref(s))
        return z, s.value, secs

    def mlp_train_f32(self, dims, weights, biases, x, y, steps, lr=1e-3):
        """Trains the tanh MLP with the reference's nn/optim classes; updates weights/biases in place.
        Returns (losses, seconds)."""
        n = len(dims) - 1
        cdims = (ctypes.c_size_t * len(dims))(*dims)
        wp = (ctypes.c_void_p * n)(*[w.ctypes.data for w in weights])
        bp = (ctypes.c_void_p * n)(*[b.ctypes.data for b in biases])
        losses = np.zeros(steps, dtype=np.float32)
        secs = self._lib.aixref_mlp_train_f32(cdims, n, x.shape[0], wp, bp, x.ctypes.data, y.ctypes.data, steps, lr, losses.ctypes.data)
        return losses, secs
