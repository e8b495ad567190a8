// Shared plain-data types of the B200 device: element types, tensor views, status-carrying exception.
#pragma once

#include "../../include/aixb200.h"

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace aixb200
{

// Error that carries the C-ABI status code it maps to.
struct Error : std::runtime_error
{
    int code;
    Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};

[[noreturn]] inline void failInvalid(const std::string& what) { throw Error(AIXB200_ERR_INVALID, what); }
[[noreturn]] inline void failRuntime(const std::string& what) { throw Error(AIXB200_ERR_RUNTIME, what); }

enum DType : uint8_t { F64 = 0, F32 = 1, F16 = 2, BF16 = 3, I64 = 4, I32 = 5, I16 = 6, I8 = 7, U8 = 8, DTYPE_COUNT = 9 };

// Element sizes; same table as aix::Device::dataTypeSize (aixDeviceCPU.cpp:685-700).
inline size_t dtypeSize(uint32_t dt)
{
    static const size_t sizes[DTYPE_COUNT] = {8, 4, 2, 2, 8, 4, 2, 1, 1};
    if (dt >= DTYPE_COUNT) failInvalid("unknown data type " + std::to_string(dt));
    return sizes[dt];
}
inline bool isFloatType(uint32_t dt) { return dt <= BF16; }
inline const char* dtypeName(uint32_t dt)
{
    static const char* names[DTYPE_COUNT] = {"f64", "f32", "f16", "bf16", "i64", "i32", "i16", "i8", "u8"};
    return dt < DTYPE_COUNT ? names[dt] : "?";
}

constexpr int MAX_RANK = AIXB200_MAX_RANK;

// A strided view into one storage. `base` is the storage base, the view begins `offset` elements in.
// Dimensions are kept collapsed: size-1 dimensions dropped and neighbours merged whenever
// stride[d] == stride[d+1] * shape[d+1], so that two descriptions of the same element sequence compare equal.
struct View
{
    char*    base = nullptr;
    uint64_t offset = 0;
    uint64_t size = 0;           // logical element count
    uint8_t  dtype = F32;
    uint8_t  rank = 0;           // collapsed rank
    uint64_t shape[MAX_RANK] = {};
    uint64_t strides[MAX_RANK] = {};

    bool isDense() const { return rank == 0 || (rank == 1 && strides[0] == 1); }     // element i lives at offset + i
    bool isBroadcastScalar() const { return rank == 0 || (rank == 1 && strides[0] == 0); }
    // Distance in elements between the first and the last element touched, plus one.
    uint64_t span() const
    {
        uint64_t s = 1;
        for (int d = 0; d < rank; ++d) s += (shape[d] - 1) * strides[d];
        return size == 0 ? 0 : s;
    }
    char* firstByte() const { return base + offset * dtypeSize(dtype); }
    char* endByte() const { return base + (offset + span()) * dtypeSize(dtype); }
    bool sameElements(const View& o) const
    {
        if (base != o.base || offset != o.offset || dtype != o.dtype || rank != o.rank || size != o.size) return false;
        for (int d = 0; d < rank; ++d)
            if (shape[d] != o.shape[d] || strides[d] != o.strides[d]) return false;
        return true;
    }
    bool overlaps(const View& o) const { return firstByte() < o.endByte() && o.firstByte() < endByte(); }
};

// Builds a collapsed View from the C descriptor; checks rank, dtype and size consistency.
inline View makeView(const aixb200_tensor* t, const char* what)
{
    if (!t) failInvalid(std::string(what) + ": null tensor descriptor");
    if (t->rank > AIXB200_MAX_RANK) failInvalid(std::string(what) + ": rank above AIXB200_MAX_RANK");
    dtypeSize(t->dtype);
    View v;
    v.base = static_cast<char*>(t->data);
    v.offset = t->offset;
    v.dtype = static_cast<uint8_t>(t->dtype);
    uint64_t n = 1;
    for (uint32_t d = 0; d < t->rank; ++d) n *= t->shape[d];
    if (t->size != n) failInvalid(std::string(what) + ": size does not match shape");
    v.size = n;
    if (n == 0) return v;
    if (!t->data) failInvalid(std::string(what) + ": null data pointer");
    for (uint32_t d = 0; d < t->rank; ++d)
    {
        uint64_t extent = t->shape[d], stride = t->strides[d];
        if (extent == 1) continue;
        if (v.rank > 0 && v.strides[v.rank - 1] == stride * extent)
        {
            v.shape[v.rank - 1] *= extent;
            v.strides[v.rank - 1] = stride;
        }
        else
        {
            v.shape[v.rank] = extent;
            v.strides[v.rank] = stride;
            ++v.rank;
        }
    }
    return v;
}

// 64-bit container for one scalar already converted to its target element type.
union ScalarBits
{
    double   f64;
    float    f32;
    uint16_t u16;
    int64_t  i64;
    int32_t  i32;
    int16_t  i16;
    int8_t   i8;
    uint8_t  u8;
    uint64_t raw;
};

// 64-bit FNV-1a, used for kernel-cache keys and cubin file names.
inline uint64_t fnv1a(const void* data, size_t len, uint64_t h = 1469598103934665603ull)
{
    auto p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < len; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}

}   // namespace aixb200
