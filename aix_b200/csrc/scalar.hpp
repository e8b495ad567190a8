// Host-side scalar conversion between the nine element types.
// Follows the reference's conversion rule for fill and dtype-converting copies
// (convertGenericValue, aixDeviceCPU.cpp:96-117): float-like -> integer saturates and maps NaN to 0,
// everything else is a plain C++ conversion; float -> bfloat16 / float16 rounds to nearest even
// (aixFloat16.hpp:775-805 and :540-620).
#pragma once

#include "common.hpp"

#include <algorithm>
#include <cmath>
#include <limits>

namespace aixb200
{

inline float bf16ToFloat(uint16_t h)
{
    uint32_t bits = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t floatToBf16(float f)
{
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu) != 0)
        return static_cast<uint16_t>((bits >> 16) | 0x0040u);                 // keep NaN a NaN
    uint32_t rounding = 0x7FFFu + ((bits >> 16) & 1u);
    return static_cast<uint16_t>((bits + rounding) >> 16);
}

inline float f16ToFloat(uint16_t h)
{
    uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0)
    {
        if (man == 0) bits = sign;
        else
        {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            bits = sign | ((113 - shift) << 23) | (man << 13);
        }
    }
    else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t floatToF16(float f)
{
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    uint16_t sign = static_cast<uint16_t>((bits >> 16) & 0x8000u);
    uint32_t abs = bits & 0x7FFFFFFFu;
    if (abs >= 0x7F800000u) return sign | (abs > 0x7F800000u ? 0x7E00u : 0x7C00u);
    if (abs >= 0x477FF000u) return sign | 0x7C00u;                            // rounds to infinity
    if (abs < 0x33000001u) return sign;                                       // rounds to zero (<= 2^-25)
    int32_t exp = static_cast<int32_t>(abs >> 23) - 127;
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
    uint32_t shift = exp < -14 ? static_cast<uint32_t>(13 + (-14 - exp)) : 13u;
    uint32_t half = man >> shift, rest = man & ((1u << shift) - 1u), mid = 1u << (shift - 1);
    if (rest > mid || (rest == mid && (half & 1u))) ++half;
    if (exp < -14) return sign | static_cast<uint16_t>(half);                 // subnormal (may carry into normal)
    return sign | static_cast<uint16_t>(((exp + 15) << 10) + (half - 0x400u));
}

// Reads one scalar of type `dt` as long double (exact for every element type).
inline long double loadScalar(const void* p, uint32_t dt)
{
    switch (dt)
    {
        case F64:  { double v;   std::memcpy(&v, p, 8); return v; }
        case F32:  { float v;    std::memcpy(&v, p, 4); return v; }
        case F16:  { uint16_t v; std::memcpy(&v, p, 2); return f16ToFloat(v); }
        case BF16: { uint16_t v; std::memcpy(&v, p, 2); return bf16ToFloat(v); }
        case I64:  { int64_t v;  std::memcpy(&v, p, 8); return v; }
        case I32:  { int32_t v;  std::memcpy(&v, p, 4); return v; }
        case I16:  { int16_t v;  std::memcpy(&v, p, 2); return v; }
        case I8:   { int8_t v;   std::memcpy(&v, p, 1); return v; }
        case U8:   { uint8_t v;  std::memcpy(&v, p, 1); return v; }
    }
    failInvalid("unknown scalar type");
}

template <typename I>
inline I saturateToInt(long double v)
{
    if (std::isnan(v)) return 0;
    v = std::clamp(v, static_cast<long double>(std::numeric_limits<I>::lowest()),
                      static_cast<long double>(std::numeric_limits<I>::max()));
    return static_cast<I>(v);
}

// Converts one host scalar of type `srcDt` into the bit pattern of type `dstDt`.
inline ScalarBits convertScalar(const void* p, uint32_t srcDt, uint32_t dstDt)
{
    ScalarBits out;
    out.raw = 0;
    const bool srcFloat = isFloatType(srcDt);
    if (!srcFloat && !isFloatType(dstDt))
    {
        // integer -> integer: two's complement truncation like static_cast
        int64_t v = (srcDt == I64) ? *static_cast<const int64_t*>(p) : static_cast<int64_t>(loadScalar(p, srcDt));
        switch (dstDt)
        {
            case I64: out.i64 = v; break;
            case I32: out.i32 = static_cast<int32_t>(v); break;
            case I16: out.i16 = static_cast<int16_t>(v); break;
            case I8:  out.i8  = static_cast<int8_t>(v); break;
            case U8:  out.u8  = static_cast<uint8_t>(v); break;
        }
        return out;
    }
    long double v = loadScalar(p, srcDt);
    switch (dstDt)
    {
        case F64:  out.f64 = static_cast<double>(v); break;
        // 16-bit float sources and f32 go through float exactly; f64 and integers round once to float first,
        // which is what static_cast<float16_t/bfloat16_t>(x) does in the reference (their only constructor is float).
        case F32:  out.f32 = (srcDt == F64) ? static_cast<float>(static_cast<double>(v)) : static_cast<float>(v); break;
        case F16:  out.u16 = floatToF16(static_cast<float>(v)); break;
        case BF16: out.u16 = floatToBf16(static_cast<float>(v)); break;
        case I64:  out.i64 = saturateToInt<int64_t>(v); break;
        case I32:  out.i32 = saturateToInt<int32_t>(v); break;
        case I16:  out.i16 = saturateToInt<int16_t>(v); break;
        case I8:   out.i8  = saturateToInt<int8_t>(v); break;
        case U8:   out.u8  = saturateToInt<uint8_t>(v); break;
        default: failInvalid("unknown scalar type");
    }
    return out;
}

// lowest() of each element type as stored bits (fillMin; aixDeviceCPU.cpp:131-138, aixFloat16.hpp lowest()).
inline ScalarBits lowestValue(uint32_t dt)
{
    ScalarBits out;
    out.raw = 0;
    switch (dt)
    {
        case F64:  out.f64 = std::numeric_limits<double>::lowest(); break;
        case F32:  out.f32 = std::numeric_limits<float>::lowest(); break;
        case F16:  out.u16 = 0xFBFFu; break;
        case BF16: out.u16 = 0xFF7Fu; break;
        case I64:  out.i64 = std::numeric_limits<int64_t>::lowest(); break;
        case I32:  out.i32 = std::numeric_limits<int32_t>::lowest(); break;
        case I16:  out.i16 = std::numeric_limits<int16_t>::lowest(); break;
        case I8:   out.i8  = std::numeric_limits<int8_t>::lowest(); break;
        case U8:   out.u8  = 0; break;
        default: failInvalid("unknown element type");
    }
    return out;
}

}   // namespace aixb200
