"""Host-side mirror of aix::TensorValue: the caller of the device interface.

It exists so that tests and benchmarks issue the SAME sequence of device calls the reference's core issues for an
expression (Targets/AIXLib/aixCore.hpp:242-1787): every operator allocates its result from the device, then makes
exactly one device call; scalars become filled tensors; broadcasting and transposition are stride-only views;
storages are released when the last view dies. It works with any object that has the aix::Device methods (the
B200 device, or the CPU oracles used by the tests) and does no arithmetic itself.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np

from . import _capi as C
from .device import DeviceTensorParams, from_storage, to_storage

# aix::promoteDataType (aixCore.hpp:71-101) and promoteDataTypeToFloat (:104-116)
_PROMOTE = [
    [0, 0, 0, 0, 0, 0, 0, 0, 0],
    [0, 1, 1, 1, 1, 1, 1, 1, 1],
    [0, 1, 2, 1, 2, 2, 2, 2, 2],
    [0, 1, 1, 3, 3, 3, 3, 3, 3],
    [0, 1, 2, 3, 4, 4, 4, 4, 4],
    [0, 1, 2, 3, 4, 5, 5, 5, 5],
    [0, 1, 2, 3, 4, 5, 6, 6, 6],
    [0, 1, 2, 3, 4, 5, 6, 7, 6],
    [0, 1, 2, 3, 4, 5, 6, 6, 8],
]
_TO_FLOAT = [0, 1, 2, 3, 1, 1, 1, 1, 1]


def promote(a: int, b: int) -> int:
    return _PROMOTE[a][b]


_STRIDES: dict = {}


def contiguous_strides(shape: Sequence[int]) -> tuple:
    shape = tuple(shape)
    known = _STRIDES.get(shape)
    if known is None:
        strides, acc = [], 1
        for s in reversed(shape):
            strides.append(acc)
            acc *= s
        known = tuple(reversed(strides))
        if len(_STRIDES) < 4096:
            _STRIDES[shape] = known
    return known


def numel(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


class TensorStorage:
    """aix::TensorStorage (aixCore.hpp:206-239): owns one device allocation."""

    def __init__(self, device, count: int, dtype: int):
        self.device = device
        self.data = device.allocate(count, dtype)
        self.count = count

    def __del__(self):
        try:
            if self.data is not None:
                self.device.deallocate(self.data)
        except Exception:
            pass


class TensorValue:
    def __init__(self, storage: TensorStorage, shape, strides, offset: int, dtype: int, device):
        self.storage, self.shape, self.strides = storage, tuple(shape), tuple(strides)
        self.offset, self.dtype, self.device = offset, dtype, device

    # ---- construction (aixCore.hpp:249-334) -------------------------------------------------------------------
    @staticmethod
    def empty(shape, device, dtype: int = C.F32) -> "TensorValue":
        shape = tuple(shape)
        return TensorValue(TensorStorage(device, numel(shape), dtype), shape, contiguous_strides(shape), 0, dtype, device)

    @staticmethod
    def full(value: float, shape, device, dtype: int = C.F32) -> "TensorValue":
        t = TensorValue.empty(shape, device, dtype)
        device.fill(value, C.F32, t.deviceParams())
        return t

    @staticmethod
    def from_numpy(values: np.ndarray, device, dtype: int = C.F32, src_dtype: int | None = None) -> "TensorValue":
        """Host data -> device tensor through Device::copy, like the host-pointer constructor."""
        src_dtype = dtype if src_dtype is None else src_dtype
        raw = to_storage(np.asarray(values), src_dtype)
        t = TensorValue.empty(np.asarray(values).shape, device, dtype)
        device.copy(raw.ctypes.data, src_dtype, t.storage.data, dtype, raw.size)
        t._host_source = raw        # keeps the host buffer alive until the copy has certainly happened
        return t

    # ---- accessors -------------------------------------------------------------------------------------------
    @property
    def size(self) -> int:
        return numel(self.shape)

    def deviceParams(self) -> DeviceTensorParams:
        p = self.__dict__.get("_params")
        if p is None or p.data != self.storage.data:
            p = DeviceTensorParams(self.storage.data, self.dtype, self.offset, self.shape, self.size, self.strides)
            self.__dict__["_params"] = p
        return p

    def isContiguous(self) -> bool:
        return self.strides == contiguous_strides(self.shape)

    def shallowCopy(self) -> "TensorValue":
        return TensorValue(self.storage, self.shape, self.strides, self.offset, self.dtype, self.device)

    def numpy(self) -> np.ndarray:
        """Synchronises and returns the logical contents as ordinary numpy numbers (bf16 as float32)."""
        t = self if (self.isContiguous() and self.offset == 0) else self.contiguous()
        self.device.synchronize()
        raw = t.device.download(t.storage.data, t.dtype, t.size)
        return from_storage(raw, t.dtype).reshape(t.shape)

    def raw(self) -> np.ndarray:
        """Storage bits (bf16/f16 as uint16/float16) of the logical contents."""
        t = self if (self.isContiguous() and self.offset == 0) else self.contiguous()
        self.device.synchronize()
        return t.device.download(t.storage.data, t.dtype, t.size).reshape(t.shape)

    def item(self):
        return self.numpy().reshape(-1)[0]

    # ---- views (aixCore.hpp:599-629, 979-994) ------------------------------------------------------------------
    def broadcastTo(self, new_shape) -> "TensorValue":
        new_shape = tuple(new_shape)
        if self.shape == new_shape:
            return self.shallowCopy()
        strides = [0] * len(new_shape)
        i = len(self.shape) - 1
        for j in range(len(new_shape) - 1, -1, -1):
            if i >= 0:
                if self.shape[i] == new_shape[j]:
                    strides[j] = self.strides[i]
                elif self.shape[i] != 1:
                    raise ValueError("Target TensorValue shape is not broadcastable.")
            i -= 1
        if i >= 0:
            raise ValueError("Target TensorValue shape is not broadcastable.")
        return TensorValue(self.storage, new_shape, strides, self.offset, self.dtype, self.device)

    def transpose(self, dim0: int, dim1: int) -> "TensorValue":
        shape, strides = list(self.shape), list(self.strides)
        shape[dim0], shape[dim1] = shape[dim1], shape[dim0]
        strides[dim0], strides[dim1] = strides[dim1], strides[dim0]
        return TensorValue(self.storage, shape, strides, self.offset, self.dtype, self.device)

    def reshape(self, new_shape) -> "TensorValue":
        new_shape = tuple(new_shape)
        if numel(new_shape) != self.size:
            raise ValueError("Reshape error: element count mismatch")
        t = self if self.isContiguous() else self.contiguous()
        return TensorValue(t.storage, new_shape, contiguous_strides(new_shape), t.offset, t.dtype, t.device)

    def squeeze(self, dim: int) -> "TensorValue":
        shape, strides = list(self.shape), list(self.strides)
        if shape[dim] == 1:
            del shape[dim], strides[dim]
        return TensorValue(self.storage, shape, strides, self.offset, self.dtype, self.device)

    def select(self, dim: int, index: int) -> "TensorValue":
        shape, strides = list(self.shape), list(self.strides)
        offset = self.offset + index * strides[dim]
        del shape[dim], strides[dim]
        return TensorValue(self.storage, shape, strides, offset, self.dtype, self.device)

    def contiguous(self) -> "TensorValue":
        if self.isContiguous() and self.offset == 0:
            return self.shallowCopy()
        result = TensorValue.empty(self.shape, self.device, self.dtype)
        self.device.contiguous(self.deviceParams(), result.deviceParams())
        return result

    def to(self, dtype: int) -> "TensorValue":
        """aixCore.hpp:530-538: conversion goes through the host-pointer constructor, i.e. Device::copy."""
        if dtype == self.dtype:
            return self.shallowCopy()
        m = self if (self.isContiguous() and self.offset == 0) else self.contiguous()
        result = TensorValue.empty(m.shape, self.device, dtype)
        self.device.copy(m.storage.data, m.dtype, result.storage.data, dtype, m.size)
        result._source = m
        return result

    # ---- arithmetic (aixCore.hpp:659-777, 1413-1470, 1616-1638) -------------------------------------------------
    @staticmethod
    def _prepare(lhs: "TensorValue", rhs: "TensorValue"):
        dtype = lhs.dtype
        if lhs.dtype != rhs.dtype:
            dtype = promote(lhs.dtype, rhs.dtype)
            lhs, rhs = lhs.to(dtype), rhs.to(dtype)
        if lhs.shape != rhs.shape:
            shape = tuple(np.broadcast_shapes(lhs.shape, rhs.shape))
            lhs, rhs = lhs.broadcastTo(shape), rhs.broadcastTo(shape)
        return lhs, rhs, TensorValue.empty(lhs.shape, lhs.device, dtype)

    def _arith(self, name: str, other) -> "TensorValue":
        if not isinstance(other, TensorValue):
            other = TensorValue.full(float(other), self.shape, self.device, _TO_FLOAT[self.dtype])
        lhs, rhs, result = TensorValue._prepare(self, other)
        getattr(self.device, name)(lhs.deviceParams(), rhs.deviceParams(), result.deviceParams())
        return result

    def _rarith(self, name: str, scalar: float) -> "TensorValue":
        return TensorValue.full(float(scalar), self.shape, self.device, _TO_FLOAT[self.dtype])._arith(name, self)

    def _inplace(self, name: str, other) -> "TensorValue":
        if not isinstance(other, TensorValue):
            other = TensorValue.full(float(other), self.shape, self.device, _TO_FLOAT[self.dtype])
        rhs = other.to(self.dtype) if other.dtype != self.dtype else other
        if rhs.shape != self.shape:
            lhs, rhs, result = TensorValue._prepare(self, rhs)
            getattr(self.device, name)(lhs.deviceParams(), rhs.deviceParams(), result.deviceParams())
            self.__dict__.update(result.__dict__)
            self.__dict__.pop("_params", None)
            return self
        getattr(self.device, name)(self.deviceParams(), rhs.deviceParams(), self.deviceParams())
        return self

    def __add__(self, o):  return self._arith("add", o)
    def __sub__(self, o):  return self._arith("sub", o)
    def __mul__(self, o):  return self._arith("mul", o)
    def __truediv__(self, o):  return self._arith("div", o)
    def __radd__(self, s): return self._rarith("add", s)
    def __rsub__(self, s): return self._rarith("sub", s)
    def __rmul__(self, s): return self._rarith("mul", s)
    def __rtruediv__(self, s): return self._rarith("div", s)
    def __iadd__(self, o): return self._inplace("add", o)
    def __isub__(self, o): return self._inplace("sub", o)
    def __imul__(self, o): return self._inplace("mul", o)
    def __itruediv__(self, o): return self._inplace("div", o)

    def __neg__(self) -> "TensorValue":
        result = TensorValue.empty(self.shape, self.device, self.dtype)
        self.device.unary(self.deviceParams(), result.deviceParams())
        return result

    def fill(self, value: float):
        self.device.fill(value, C.F32, self.deviceParams())

    def _math(self, name: str) -> "TensorValue":
        """tensorMathFunc (aixCore.hpp:1452-1468): integers are first copied to float32, then updated in place."""
        promoted = _TO_FLOAT[self.dtype]
        if promoted != self.dtype:
            result = self.to(promoted)
            getattr(self.device, name)(result.deviceParams(), result.deviceParams())
            return result
        result = TensorValue.empty(self.shape, self.device, self.dtype)
        getattr(self.device, name)(self.deviceParams(), result.deviceParams())
        return result

    def sqrt(self): return self._math("sqrt")
    def sin(self):  return self._math("sin")
    def cos(self):  return self._math("cos")
    def tanh(self): return self._math("tanh")
    def log(self):  return self._math("log")
    def exp(self):  return self._math("exp")

    def pow(self, exponent: "TensorValue") -> "TensorValue":
        lhs, rhs, result = TensorValue._prepare(self, exponent)
        self.device.pow(lhs.deviceParams(), rhs.deviceParams(), result.deviceParams())
        return result

    # ---- reductions (aixCore.hpp:632-639, 784-891) -------------------------------------------------------------
    def sum(self, dim: int | None = None, keepDim: bool = False) -> "TensorValue":
        if dim is None:
            result = TensorValue.empty((), self.device, self.dtype)
            self.device.sum(self.deviceParams(), result.deviceParams())
            return result
        dim = dim + len(self.shape) if dim < 0 else dim
        shape = list(self.shape)
        shape[dim] = 1
        result = self.reduceTo(shape)
        return result if keepDim else result.squeeze(dim)

    def reduceTo(self, shape) -> "TensorValue":
        if tuple(shape) == self.shape:
            return self.shallowCopy()
        result = TensorValue.full(0, shape, self.device, self.dtype)
        self.device.reduceTo(self.deviceParams(), result.deviceParams())
        return result

    def mean(self) -> "TensorValue":
        return self.sum() / float(self.size)

    def max(self, dim: int | None = None, keepDim: bool = False) -> "TensorValue":
        if dim is None:
            result = TensorValue.empty((), self.device, self.dtype)
            self.device.max(self.deviceParams(), result.deviceParams())
            return result
        dim = dim + len(self.shape) if dim < 0 else dim
        shape = list(self.shape)
        shape[dim] = 1
        result = TensorValue.empty(shape, self.device, self.dtype)
        self.device.fillMin(result.deviceParams())
        self.device.maxTo(self.deviceParams(), result.deviceParams())
        return result if keepDim else result.squeeze(dim)

    def matmul(self, b: "TensorValue") -> "TensorValue":
        if len(self.shape) != 2 or len(b.shape) != 2:
            raise ValueError("Both tensors must be 2D for matrix multiplication.")
        if self.shape[1] != b.shape[0]:
            raise ValueError("The inner dimensions of the tensors do not match.")
        lhs, rhs = self, b
        if lhs.dtype != rhs.dtype:
            dtype = promote(lhs.dtype, rhs.dtype)
            lhs, rhs = lhs.to(dtype), rhs.to(dtype)
        result = TensorValue.empty((self.shape[0], b.shape[1]), self.device, lhs.dtype)
        self.device.matmul(lhs.deviceParams(), rhs.deviceParams(), result.deviceParams())
        return result


def scalar_like(value: float, like: TensorValue) -> TensorValue:
    """The aix::Tensor-level scalar operand (aixCore.hpp:2384-2438): a one-element tensor filled on the device and
    broadcast with zero strides to the other operand's shape."""
    one = TensorValue.full(value, (), like.device, _TO_FLOAT[like.dtype])
    return one.broadcastTo(like.shape)
