// Device-side element-type traits for the fixed kernels (reductions, GEMM fallback, data movement).
// Rounding and wrap-around rules are those of the reference's CPU device: f16/bf16 convert through float with
// round-to-nearest-even (aixFloat16.hpp:104-122, 698-716, 775-805), integers wrap in their storage type.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace aixb200::dev
{

__device__ __forceinline__ float f16ToF32(uint16_t h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ uint16_t f32ToF16(float f) { uint16_t h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float bf16ToF32(uint16_t h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }
__device__ __forceinline__ uint16_t f32ToBf16(float f) { uint16_t h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }

// S: storage type. V: value type used for arithmetic and comparisons (exact image of S).
// SumA: per-thread sum accumulator. SumW / MaxW: 64-bit types used when combining across threads and blocks.
template <int DT> struct Elem;

template <> struct Elem<0> { typedef double S; typedef double V; typedef double SumA; typedef double SumW; typedef double MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return v; }
    static __device__ __forceinline__ S fromSum(SumW w) { return w; } static __device__ __forceinline__ V lowest() { return -INFINITY; } };
template <> struct Elem<1> { typedef float S; typedef float V; typedef float SumA; typedef double SumW; typedef double MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return v; }
    static __device__ __forceinline__ S fromSum(SumW w) { return static_cast<float>(w); } static __device__ __forceinline__ V lowest() { return -INFINITY; } };
template <> struct Elem<2> { typedef uint16_t S; typedef float V; typedef float SumA; typedef double SumW; typedef double MaxW;
    static __device__ __forceinline__ V load(S s) { return f16ToF32(s); }   static __device__ __forceinline__ S store(V v) { return f32ToF16(v); }
    static __device__ __forceinline__ S fromSum(SumW w) { return f32ToF16(static_cast<float>(w)); } static __device__ __forceinline__ V lowest() { return -INFINITY; } };
template <> struct Elem<3> { typedef uint16_t S; typedef float V; typedef float SumA; typedef double SumW; typedef double MaxW;
    static __device__ __forceinline__ V load(S s) { return bf16ToF32(s); }   static __device__ __forceinline__ S store(V v) { return f32ToBf16(v); }
    static __device__ __forceinline__ S fromSum(SumW w) { return f32ToBf16(static_cast<float>(w)); } static __device__ __forceinline__ V lowest() { return -INFINITY; } };
template <> struct Elem<4> { typedef int64_t S; typedef int64_t V; typedef uint64_t SumA; typedef uint64_t SumW; typedef int64_t MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return v; }
    static __device__ __forceinline__ S fromSum(SumW w) { return static_cast<int64_t>(w); } static __device__ __forceinline__ V lowest() { return INT64_MIN; } };
template <> struct Elem<5> { typedef int32_t S; typedef int32_t V; typedef uint32_t SumA; typedef uint64_t SumW; typedef int64_t MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return v; }
    static __device__ __forceinline__ S fromSum(SumW w) { return static_cast<int32_t>(static_cast<uint32_t>(w)); } static __device__ __forceinline__ V lowest() { return INT32_MIN; } };
template <> struct Elem<6> { typedef int16_t S; typedef int32_t V; typedef uint32_t SumA; typedef uint64_t SumW; typedef int64_t MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return static_cast<int16_t>(v); }
    static __device__ __forceinline__ S fromSum(SumW w) { return static_cast<int16_t>(static_cast<uint32_t>(w)); } static __device__ __forceinline__ V lowest() { return -32768; } };
template <> struct Elem<7> { typedef int8_t S; typedef int32_t V; typedef uint32_t SumA; typedef uint64_t SumW; typedef int64_t MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return static_cast<int8_t>(v); }
    static __device__ __forceinline__ S fromSum(SumW w) { return static_cast<int8_t>(static_cast<uint32_t>(w)); } static __device__ __forceinline__ V lowest() { return -128; } };
template <> struct Elem<8> { typedef uint8_t S; typedef int32_t V; typedef uint32_t SumA; typedef uint64_t SumW; typedef int64_t MaxW;
    static __device__ __forceinline__ V load(S s) { return s; }   static __device__ __forceinline__ S store(V v) { return static_cast<uint8_t>(v); }
    static __device__ __forceinline__ S fromSum(SumW w) { return static_cast<uint8_t>(static_cast<uint32_t>(w)); } static __device__ __forceinline__ V lowest() { return 0; } };

template <class S, int N> struct alignas(sizeof(S) * N >= 16 ? 16 : sizeof(S) * N) Pack { S v[N]; };

// Reduction policy: sum or max over element type DT.
template <int DT, bool IsMax> struct Reduce;

template <int DT> struct Reduce<DT, false>
{
    typedef Elem<DT> E; typedef typename E::S S; typedef typename E::SumA A; typedef typename E::SumW W;
    static __device__ __forceinline__ A init() { return A(0); }
    static __device__ __forceinline__ A step(A acc, S s) { return acc + static_cast<A>(E::load(s)); }
    static __device__ __forceinline__ W widen(A a) { return static_cast<W>(a); }
    static __device__ __forceinline__ W identityW() { return W(0); }
    static __device__ __forceinline__ W merge(W a, W b) { return a + b; }
    static __device__ __forceinline__ W liftStored(S s) { return static_cast<W>(static_cast<A>(E::load(s))); }
    static __device__ __forceinline__ S finish(W w) { return E::fromSum(w); }
};

template <int DT> struct Reduce<DT, true>
{
    typedef Elem<DT> E; typedef typename E::S S; typedef typename E::V A; typedef typename E::MaxW W;
    static __device__ __forceinline__ A init() { return E::lowest(); }
    static __device__ __forceinline__ A step(A acc, S s) { A v = E::load(s); return v > acc ? v : acc; }
    static __device__ __forceinline__ W widen(A a) { return static_cast<W>(a); }
    static __device__ __forceinline__ W identityW() { return static_cast<W>(E::lowest()); }
    static __device__ __forceinline__ W merge(W a, W b) { return b > a ? b : a; }
    static __device__ __forceinline__ W liftStored(S s) { return static_cast<W>(E::load(s)); }
    static __device__ __forceinline__ S finish(W w) { return E::store(static_cast<typename E::V>(w)); }
};

template <class W> __device__ __forceinline__ W shuffleDown(W v, int delta)
{
    static_assert(sizeof(W) == 8, "cross-thread values are 64-bit");
    long long bits = __shfl_down_sync(0xffffffffu, *reinterpret_cast<long long*>(&v), delta);
    return *reinterpret_cast<W*>(&bits);
}

// Block-wide reduction of one W per thread; the result is valid in thread 0. `smem` holds 32 W.
template <class R> __device__ __forceinline__ typename R::W blockReduce(typename R::W v, typename R::W* smem)
{
    typedef typename R::W W;
    #pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = R::merge(v, shuffleDown<W>(v, d));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    __syncthreads();                       // smem may still be read by a previous use
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0)
    {
        v = lane < warps ? smem[lane] : R::identityW();
        #pragma unroll
        for (int d = 16; d > 0; d >>= 1) v = R::merge(v, shuffleDown<W>(v, d));
    }
    return v;
}

}   // namespace aixb200::dev

// Calls F<DT>(args...) for the runtime element type `dt`.
#define AIXB200_DISPATCH_DTYPE(dt, F, ...)                                   \
    switch (dt)                                                              \
    {                                                                        \
        case 0: F<0>(__VA_ARGS__); break;                                    \
        case 1: F<1>(__VA_ARGS__); break;                                    \
        case 2: F<2>(__VA_ARGS__); break;                                    \
        case 3: F<3>(__VA_ARGS__); break;                                    \
        case 4: F<4>(__VA_ARGS__); break;                                    \
        case 5: F<5>(__VA_ARGS__); break;                                    \
        case 6: F<6>(__VA_ARGS__); break;                                    \
        case 7: F<7>(__VA_ARGS__); break;                                    \
        case 8: F<8>(__VA_ARGS__); break;                                    \
        default: break;                                                      \
    }
