#include "codegen.hpp"

#include <algorithm>
#include <sstream>

namespace aixb200
{

namespace
{

// Element-type traits and per-op semantics shared by every generated kernel.
//
// Semantics follow the reference's CPU device (aixDeviceCPU.cpp:28-255):
//  * f16 / bf16 compute every op in float and round to the 16-bit type after it (aixFloat16.hpp:104-122, 698-716);
//  * integers wrap in their storage type; 8/16-bit values are held in int and re-narrowed after each op;
//  * sqrt/log/exp/pow on integers go through a wide float and a saturating, NaN->0 conversion back
//    (convertGenericValue, aixDeviceCPU.cpp:96-117); sin/cos/tanh on integers are a plain truncating conversion;
//  * dtype conversion float-like -> integer saturates and maps NaN to 0, everything else is a C++ static_cast.
const char* kPrelude = R"PRELUDE(
typedef unsigned short     u16_t;
typedef long long          i64_t;
typedef unsigned long long u64_t;

template <class S, int E> struct alignas((sizeof(S) * E) >= 16 ? 16 : (sizeof(S) * E)) Pack { S v[E]; };

__device__ __forceinline__ float f16_to_f32(u16_t h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16_t f32_to_f16(float f) { u16_t h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float bf16_to_f32(u16_t h) { return __uint_as_float(((unsigned)h) << 16); }
__device__ __forceinline__ u16_t f32_to_bf16(float f) { u16_t h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }

// kind: 0 = IEEE float computed in C, 1 = integer (wraps; C is the register type, U its unsigned twin)
struct Df64  { typedef double S; typedef double C; typedef double U; static const int kind = 0; static const int id = 0;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return c; }
    static __device__ __forceinline__ C fix(C c) { return c; } };
struct Df32  { typedef float S; typedef float C; typedef float U; static const int kind = 0; static const int id = 1;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return c; }
    static __device__ __forceinline__ C fix(C c) { return c; } };
struct Df16  { typedef u16_t S; typedef float C; typedef float U; static const int kind = 0; static const int id = 2;
    static __device__ __forceinline__ C ld(S s) { return f16_to_f32(s); }  static __device__ __forceinline__ S st(C c) { return f32_to_f16(c); }
    static __device__ __forceinline__ C fix(C c) { return f16_to_f32(f32_to_f16(c)); } };
struct Dbf16 { typedef u16_t S; typedef float C; typedef float U; static const int kind = 0; static const int id = 3;
    static __device__ __forceinline__ C ld(S s) { return bf16_to_f32(s); }  static __device__ __forceinline__ S st(C c) { return f32_to_bf16(c); }
    static __device__ __forceinline__ C fix(C c) { return bf16_to_f32(f32_to_bf16(c)); } };
struct Di64  { typedef i64_t S; typedef i64_t C; typedef u64_t U; static const int kind = 1; static const int id = 4;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return c; }
    static __device__ __forceinline__ C fix(C c) { return c; }
    static __device__ __forceinline__ C sat(double x) { return __double2ll_rz(x); } };
struct Di32  { typedef int S; typedef int C; typedef unsigned U; static const int kind = 1; static const int id = 5;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return c; }
    static __device__ __forceinline__ C fix(C c) { return c; }
    static __device__ __forceinline__ C sat(double x) { return __double2int_rz(x); } };
struct Di16  { typedef short S; typedef int C; typedef unsigned U; static const int kind = 1; static const int id = 6;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return (short)c; }
    static __device__ __forceinline__ C fix(C c) { return (int)(short)c; }
    static __device__ __forceinline__ C sat(double x) { return min(max(__double2int_rz(x), -32768), 32767); } };
struct Di8   { typedef signed char S; typedef int C; typedef unsigned U; static const int kind = 1; static const int id = 7;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return (signed char)c; }
    static __device__ __forceinline__ C fix(C c) { return (int)(signed char)c; }
    static __device__ __forceinline__ C sat(double x) { return min(max(__double2int_rz(x), -128), 127); } };
struct Du8   { typedef unsigned char S; typedef int C; typedef unsigned U; static const int kind = 1; static const int id = 8;
    static __device__ __forceinline__ C ld(S s) { return s; }  static __device__ __forceinline__ S st(C c) { return (unsigned char)c; }
    static __device__ __forceinline__ C fix(C c) { return (int)(unsigned char)c; }
    static __device__ __forceinline__ C sat(double x) { return min(max(__double2int_rz(x), 0), 255); } };

// AIX_FAST selects cheaper float routines whose error stays below 1e-6 relative (division and square root come from
// the compiler flags --prec-div=false / --prec-sqrt=false; exp and tanh below). sin, cos, log and pow keep the
// accurate library versions in both modes: their fast forms lose relative accuracy near zeros and near 1.
#if AIX_FAST
__device__ __forceinline__ float fast_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float fast_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float fast_exp(float x) { return fast_ex2(x * 1.4426950408889634f); }
__device__ __forceinline__ float fast_tanh(float x)
{
    // |x| < 0.6: x + x^3 * p(x^2), a degree-4 fit of (tanh(x) - x) / x^3 (max relative error 9e-8);
    // otherwise 1 - 2 / (exp(2|x|) + 1) with the sign of x (saturates to +-1 for large |x|).
    const float t = fabsf(x), u = x * x;
    float p = -0.006276384927332401f;
    p = fmaf(p, u, 0.021116212010383606f);
    p = fmaf(p, u, -0.053875137120485306f);
    p = fmaf(p, u, 0.13332924246788025f);
    p = fmaf(p, u, -0.3333333134651184f);
    const float small = fmaf(x * u, p, x);
    const float e = fast_ex2(t * 2.885390081777927f);
    const float large = copysignf(fmaf(-2.0f, fast_rcp(e + 1.0f), 1.0f), x);
    return t < 0.6f ? small : large;
}
#endif

__device__ __forceinline__ float  m_sqrt(float x)  { return sqrtf(x); }   __device__ __forceinline__ double m_sqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float  m_sin(float x)   { return sinf(x); }    __device__ __forceinline__ double m_sin(double x)  { return sin(x); }
__device__ __forceinline__ float  m_cos(float x)   { return cosf(x); }    __device__ __forceinline__ double m_cos(double x)  { return cos(x); }
#if AIX_FAST
__device__ __forceinline__ float  m_tanh(float x)  { return fast_tanh(x); }
#else
__device__ __forceinline__ float  m_tanh(float x)  { return tanhf(x); }
#endif
__device__ __forceinline__ double m_tanh(double x) { return tanh(x); }
__device__ __forceinline__ float  m_log(float x)   { return logf(x); }    __device__ __forceinline__ double m_log(double x)  { return log(x); }
#if AIX_FAST
__device__ __forceinline__ float  m_exp(float x)   { return fast_exp(x); }
#else
__device__ __forceinline__ float  m_exp(float x)   { return expf(x); }
#endif
__device__ __forceinline__ double m_exp(double x)  { return exp(x); }
__device__ __forceinline__ float  m_pow(float x, float y)   { return powf(x, y); }
__device__ __forceinline__ double m_pow(double x, double y) { return pow(x, y); }

// Integer pow goes through double; the reference uses long double, whose result is exact whenever the true power is
// an integer. A last-place error of pow() must not turn 3 into 2 under truncation, so results that sit within a few
// ulps of an integer are snapped to it.
__device__ __forceinline__ double snap_integer(double r) { const double n = rint(r); return (fabs(r - n) <= fabs(n) * 8.9e-16) ? n : r; }

#define AIX_C typename D::C
#define AIX_U typename D::U
template <class D> __device__ __forceinline__ AIX_C op_add(AIX_C a, AIX_C b) { if constexpr (D::kind == 0) return D::fix(a + b); else return D::fix((AIX_C)((AIX_U)a + (AIX_U)b)); }
template <class D> __device__ __forceinline__ AIX_C op_sub(AIX_C a, AIX_C b) { if constexpr (D::kind == 0) return D::fix(a - b); else return D::fix((AIX_C)((AIX_U)a - (AIX_U)b)); }
template <class D> __device__ __forceinline__ AIX_C op_mul(AIX_C a, AIX_C b) { if constexpr (D::kind == 0) return D::fix(a * b); else return D::fix((AIX_C)((AIX_U)a * (AIX_U)b)); }
template <class D> __device__ __forceinline__ AIX_C op_div(AIX_C a, AIX_C b)
{
    if constexpr (D::kind == 0) return D::fix(a / b);
    else if constexpr (D::id == 4) return (b == 0) ? (AIX_C)0 : ((b == -1) ? (AIX_C)((AIX_U)0 - (AIX_U)a) : a / b);
    else return (b == 0) ? 0 : D::fix((AIX_C)((i64_t)a / (i64_t)b));
}
template <class D> __device__ __forceinline__ AIX_C op_neg(AIX_C a) { if constexpr (D::kind == 0) return D::fix(-a); else return D::fix((AIX_C)((AIX_U)0 - (AIX_U)a)); }
template <class D> __device__ __forceinline__ AIX_C op_sqrt(AIX_C a) { if constexpr (D::kind == 0) return D::fix(m_sqrt(a)); else return D::sat(sqrt((double)a)); }
template <class D> __device__ __forceinline__ AIX_C op_log(AIX_C a)  { if constexpr (D::kind == 0) return D::fix(m_log(a));  else return D::sat(log((double)a)); }
template <class D> __device__ __forceinline__ AIX_C op_exp(AIX_C a)  { if constexpr (D::kind == 0) return D::fix(m_exp(a));  else return D::sat(exp((double)a)); }
template <class D> __device__ __forceinline__ AIX_C op_pow(AIX_C a, AIX_C b) { if constexpr (D::kind == 0) return D::fix(m_pow(a, b)); else return D::sat(snap_integer(pow((double)a, (double)b))); }
template <class D> __device__ __forceinline__ AIX_C op_sin(AIX_C a)  { if constexpr (D::kind == 0) return D::fix(m_sin(a));  else return D::fix((AIX_C)sin((double)a)); }
template <class D> __device__ __forceinline__ AIX_C op_cos(AIX_C a)  { if constexpr (D::kind == 0) return D::fix(m_cos(a));  else return D::fix((AIX_C)cos((double)a)); }
template <class D> __device__ __forceinline__ AIX_C op_tanh(AIX_C a) { if constexpr (D::kind == 0) return D::fix(m_tanh(a)); else return D::fix((AIX_C)tanh((double)a)); }
// SD -> D conversion of a register value
template <class SD, class D> __device__ __forceinline__ AIX_C op_cast(typename SD::C x)
{
    if constexpr (SD::id == D::id) return x;
    else if constexpr (D::kind == 1 && SD::kind == 0) return D::sat((double)x);
    else if constexpr (D::kind == 1) return D::fix((AIX_C)x);
    else if constexpr (D::id == 0) return (double)x;
    else return D::fix((float)x);
}

// ---- two 16-bit floats per 32-bit register --------------------------------------------------------------------
// add / sub / mul run on the packed half-precision pipes (one instruction for two elements). Their single rounding
// equals the reference's "compute in float, round to the 16-bit type": the exact product of two 8- or 11-bit
// significands fits in float, and a float sum of two such values can only be inexact when the smaller operand lies
// entirely below the rounding position of the 16-bit result. Everything else unpacks to float, computes, and repacks
// with one round-to-nearest-even conversion for both halves.
template <class D> struct P2;
template <> struct P2<Dbf16>
{
    static __device__ __forceinline__ unsigned splat(u16_t s) { return (unsigned)s | ((unsigned)s << 16); }
    static __device__ __forceinline__ unsigned join(u16_t lo, u16_t hi) { return (unsigned)lo | ((unsigned)hi << 16); }
    static __device__ __forceinline__ float lo(unsigned p) { return __uint_as_float(p << 16); }
    static __device__ __forceinline__ float hi(unsigned p) { return __uint_as_float(p & 0xffff0000u); }
    static __device__ __forceinline__ unsigned pack(float l, float h) { unsigned d; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(h), "f"(l)); return d; }
    static __device__ __forceinline__ unsigned add(unsigned a, unsigned b) { unsigned d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ unsigned sub(unsigned a, unsigned b) { unsigned d; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ unsigned mul(unsigned a, unsigned b) { unsigned d; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
};
template <> struct P2<Df16>
{
    static __device__ __forceinline__ unsigned splat(u16_t s) { return (unsigned)s | ((unsigned)s << 16); }
    static __device__ __forceinline__ unsigned join(u16_t lo, u16_t hi) { return (unsigned)lo | ((unsigned)hi << 16); }
    static __device__ __forceinline__ float lo(unsigned p) { return f16_to_f32((u16_t)(p & 0xffffu)); }
    static __device__ __forceinline__ float hi(unsigned p) { return f16_to_f32((u16_t)(p >> 16)); }
    static __device__ __forceinline__ unsigned pack(float l, float h) { unsigned d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(h), "f"(l)); return d; }
    static __device__ __forceinline__ unsigned add(unsigned a, unsigned b) { unsigned d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ unsigned sub(unsigned a, unsigned b) { unsigned d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ unsigned mul(unsigned a, unsigned b) { unsigned d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
};
template <class D> __device__ __forceinline__ unsigned pp_add(unsigned a, unsigned b) { return P2<D>::add(a, b); }
template <class D> __device__ __forceinline__ unsigned pp_sub(unsigned a, unsigned b) { return P2<D>::sub(a, b); }
template <class D> __device__ __forceinline__ unsigned pp_mul(unsigned a, unsigned b) { return P2<D>::mul(a, b); }
template <class D> __device__ __forceinline__ unsigned pp_neg(unsigned a) { return a ^ 0x80008000u; }
template <class D> __device__ __forceinline__ unsigned pp_cast(unsigned a) { return a; }
#if AIX_FAST
// The quotient is rounded to 8 or 11 significant bits right away: a reciprocal good to 1 ulp of float is plenty.
template <class D> __device__ __forceinline__ unsigned pp_div(unsigned a, unsigned b) { return P2<D>::pack(P2<D>::lo(a) * fast_rcp(P2<D>::lo(b)), P2<D>::hi(a) * fast_rcp(P2<D>::hi(b))); }
#else
template <class D> __device__ __forceinline__ unsigned pp_div(unsigned a, unsigned b) { return P2<D>::pack(P2<D>::lo(a) / P2<D>::lo(b), P2<D>::hi(a) / P2<D>::hi(b)); }
#endif
template <class D> __device__ __forceinline__ unsigned pp_pow(unsigned a, unsigned b) { return P2<D>::pack(m_pow(P2<D>::lo(a), P2<D>::lo(b)), m_pow(P2<D>::hi(a), P2<D>::hi(b))); }
#define AIX_PP_UNARY(NAME) template <class D> __device__ __forceinline__ unsigned pp_##NAME(unsigned a) { return P2<D>::pack(m_##NAME(P2<D>::lo(a)), m_##NAME(P2<D>::hi(a))); }
AIX_PP_UNARY(sqrt) AIX_PP_UNARY(sin) AIX_PP_UNARY(cos) AIX_PP_UNARY(log) AIX_PP_UNARY(exp)
#if AIX_FAST
// bfloat16 keeps 8 significant bits: the hardware tanh (relative error 2^-11) is exact to a quarter of the last place
// of the result, so it differs from the rounded exact value by at most one bfloat16 ulp, and only near rounding ties.
__device__ __forceinline__ float hw_tanh(float x) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
template <class D> __device__ __forceinline__ unsigned pp_tanh(unsigned a)
{
    if constexpr (D::id == 3) return P2<D>::pack(hw_tanh(P2<D>::lo(a)), hw_tanh(P2<D>::hi(a)));
    else return P2<D>::pack(m_tanh(P2<D>::lo(a)), m_tanh(P2<D>::hi(a)));
}
#else
AIX_PP_UNARY(tanh)
#endif

// ---- full reductions folded into a fused kernel ---------------------------------------------------------------------
// Per thread: float (double for f64) or wrapping unsigned partial sums, the element's own register type for maxima.
// Across threads and blocks: 64-bit values, one partial per block in device scratch; the block that draws the last
// ticket folds the partials (fixed order for a fixed grid: reproducible), converts once and resets the ticket.
template <class D> __device__ __forceinline__ AIX_C red_lowest()
{
    if constexpr (D::kind == 0) return (AIX_C)(-__int_as_float(0x7f800000));
    else if constexpr (D::id == 4) return (i64_t)0x8000000000000000ull;
    else if constexpr (D::id == 5) return (int)0x80000000u;
    else if constexpr (D::id == 6) return -32768;
    else if constexpr (D::id == 7) return -128;
    else return 0;
}
template <bool B, class X, class Y> struct red_sel { typedef X T; };
template <class X, class Y> struct red_sel<false, X, Y> { typedef Y T; };
template <class D, bool IsMax> struct Red;
template <class D> struct Red<D, false>
{
    typedef typename D::S S;
    typedef typename red_sel<D::kind == 0, typename red_sel<D::id == 0, double, float>::T, typename red_sel<D::id == 4, u64_t, unsigned>::T>::T A;
    typedef typename red_sel<D::kind == 0, double, u64_t>::T W;
    static __device__ __forceinline__ A init() { return (A)0; }
    static __device__ __forceinline__ A step(A acc, AIX_C v) { return acc + (A)v; }
    static __device__ __forceinline__ W widen(A a) { return (W)a; }
    static __device__ __forceinline__ W identity() { return (W)0; }
    static __device__ __forceinline__ W merge(W a, W b) { return a + b; }
    static __device__ __forceinline__ W lift(S s) { return (W)(A)D::ld(s); }
    static __device__ __forceinline__ S finish(W w)
    {
        if constexpr (D::kind == 0 && D::id == 0) return w;
        else if constexpr (D::kind == 0) return D::st((float)w);
        else if constexpr (D::id == 4) return (i64_t)w;
        else return D::st((AIX_C)(unsigned)w);
    }
};
template <class D> struct Red<D, true>
{
    typedef typename D::S S;
    typedef AIX_C A;
    typedef typename red_sel<D::kind == 0, double, i64_t>::T W;
    static __device__ __forceinline__ A init() { return red_lowest<D>(); }
    static __device__ __forceinline__ A step(A acc, A v) { return v > acc ? v : acc; }
    static __device__ __forceinline__ W widen(A a) { return (W)a; }
    static __device__ __forceinline__ W identity() { return (W)red_lowest<D>(); }
    static __device__ __forceinline__ W merge(W a, W b) { return b > a ? b : a; }
    static __device__ __forceinline__ W lift(S s) { return (W)D::ld(s); }
    static __device__ __forceinline__ S finish(W w) { return D::st((A)w); }
};
// max|x| of f32 values as a bit pattern (non-negative floats order like unsigned integers; a NaN carries the largest
// patterns and so ends up as the maximum): the scale source of a prepared matmul operand.
struct RedAbsBits
{
    typedef unsigned S;
    typedef unsigned A;
    typedef u64_t W;
    static __device__ __forceinline__ A init() { return 0u; }
    static __device__ __forceinline__ A step(A acc, float v) { const unsigned b = __float_as_uint(fabsf(v)); return b > acc ? b : acc; }
    static __device__ __forceinline__ W widen(A a) { return (W)a; }
    static __device__ __forceinline__ W identity() { return (W)0; }
    static __device__ __forceinline__ W merge(W a, W b) { return b > a ? b : a; }
    static __device__ __forceinline__ S finish(W w) { return (unsigned)w; }
};
template <class W> __device__ __forceinline__ W red_shfl(W v, int d)
{
    i64_t bits = __shfl_down_sync(0xffffffffu, *(i64_t*)&v, d);
    return *(W*)&bits;
}
template <class R> __device__ __forceinline__ typename R::W red_block(typename R::W v, typename R::W* smem)
{
    #pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = R::merge(v, red_shfl<typename R::W>(v, d));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0)
    {
        v = lane < warps ? smem[lane] : R::identity();
        #pragma unroll
        for (int d = 16; d > 0; d >>= 1) v = R::merge(v, red_shfl<typename R::W>(v, d));
    }
    return v;
}
// Fold of one value per thread over a row's owners: the lanes of a warp (shuffles only) or the threads of the CTA.
// The result is valid in lane 0 / thread 0.
template <class R, bool WARP> __device__ __forceinline__ typename R::W row_fold(typename R::A acc, u64_t* smem)
{
    typename R::W w = R::widen(acc);
    if constexpr (WARP)
    {
        #pragma unroll
        for (int d = 16; d > 0; d >>= 1) w = R::merge(w, red_shfl<typename R::W>(w, d));
        return w;
    }
    else return red_block<R>(w, (typename R::W*)smem);
}
template <class R> __device__ __forceinline__ void red_finish(typename R::A acc, u64_t* partials, unsigned* ticket, typename R::S* out)
{
    __shared__ typename R::W smem[32];
    __shared__ bool last;
    typename R::W w = red_block<R>(R::widen(acc), smem);
    if (threadIdx.x == 0)
    {
        partials[blockIdx.x] = *(u64_t*)&w;
        __threadfence();
        last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    typename R::W total = R::identity();
    for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x)
    {
        u64_t bits = __ldcg(partials + b);
        total = R::merge(total, *(typename R::W*)&bits);
    }
    total = red_block<R>(total, smem);
    if (threadIdx.x == 0) { out[0] = R::finish(total); *ticket = 0; }
}
)PRELUDE";

const char* kTraits[DTYPE_COUNT] = {"Df64", "Df32", "Df16", "Dbf16", "Di64", "Di32", "Di16", "Di8", "Du8"};

enum class Path : uint8_t { DenseWide, DenseElem, Scalar, RowWide, ColWide, General };

Path loadPath(const KernelLoad& l, bool fast)
{
    switch (l.access)
    {
        case Access::Dense:    return fast ? Path::DenseWide : Path::DenseElem;
        case Access::Scalar:   return Path::Scalar;
        case Access::RowBcast: return fast ? Path::RowWide : Path::General;
        case Access::ColBcast: return fast ? Path::ColWide : Path::General;
        default:               return Path::General;
    }
}

Path storePath(const KernelStore& s, bool fast)
{
    if (s.access == Access::Dense) return fast ? Path::DenseWide : Path::DenseElem;
    return Path::General;
}

bool aligned(const View& v, size_t bytes) { return (reinterpret_cast<uintptr_t>(v.firstByte()) % bytes) == 0; }

size_t packBytes(uint8_t dtype, int vec) { return std::min<size_t>(16, dtypeSize(dtype) * vec); }

}   // namespace

KernelVariant chooseVariant(const KernelSpec& spec)
{
    KernelVariant v;
    size_t minSize = 8, maxSize = 1;
    uint64_t maxSpan = spec.count;
    for (auto& l : spec.loads)
    {
        if (l.access != Access::Scalar) { minSize = std::min(minSize, dtypeSize(l.view.dtype)); maxSize = std::max(maxSize, dtypeSize(l.view.dtype)); }
        maxSpan = std::max(maxSpan, l.view.span());
    }
    for (auto& s : spec.stores)
    {
        minSize = std::min(minSize, dtypeSize(s.view.dtype));
        maxSize = std::max(maxSize, dtypeSize(s.view.dtype));
        maxSpan = std::max(maxSpan, s.view.span());
    }
    v.vec = static_cast<int>(std::max<size_t>(1, std::min<size_t>(16 / minSize, 64 / maxSize)));
    v.rowMode = spec.rowCols != 0;
    if (v.rowMode)
    {
        if (spec.rowCols % static_cast<uint64_t>(v.vec) != 0) v.vec = 1;      // rows must start on a pack boundary
        const uint64_t rows = spec.count / spec.rowCols;
        v.warpPerRow = spec.rowCols * maxSize <= 65536 && rows >= 2048;
    }
    // Packed two-per-register arithmetic needs one 16-bit float type throughout the kernel.
    {
        int common = -1;
        bool uniform = true;
        auto see = [&](uint8_t dt) { if (common < 0) common = dt; else if (common != dt) uniform = false; };
        for (auto& l : spec.loads) see(l.view.dtype);
        for (auto& st : spec.stores) see(st.view.dtype);
        for (auto& nd : spec.nodes) { see(nd.dtype); if (nd.op == Op::Cast) see(nd.srcDtype); }
        v.packed16 = uniform && (common == F16 || common == BF16) && v.vec >= 2 && v.vec % 2 == 0;
    }
    v.index64 = maxSpan >= (uint64_t(1) << 31);
    for (size_t i = 0; i < spec.loads.size(); ++i)
    {
        const KernelLoad& l = spec.loads[i];
        bool fast = false;
        switch (l.access)
        {
            case Access::Dense:    fast = aligned(l.view, packBytes(l.view.dtype, v.vec)); break;
            case Access::Scalar:   fast = true; break;
            case Access::RowBcast: fast = (l.view.shape[1] % v.vec == 0) && aligned(l.view, packBytes(l.view.dtype, v.vec)) &&
                                          (!v.rowMode || l.view.shape[1] == spec.rowCols); break;
            case Access::ColBcast: fast = (l.view.shape[1] % v.vec == 0) && (!v.rowMode || l.view.shape[1] == spec.rowCols); break;
            default: break;
        }
        if (fast) v.fastLoads |= (1u << i);
    }
    for (size_t i = 0; i < spec.stores.size(); ++i)
    {
        const KernelStore& s = spec.stores[i];
        if (s.access == Access::Dense && aligned(s.view, packBytes(s.view.dtype, v.vec))) v.fastStores |= (1u << i);
    }
    return v;
}

std::string kernelKey(const KernelSpec& spec, const KernelVariant& variant, const CodegenOptions& options)
{
    std::string key;
    key.reserve(64 + spec.nodes.size() * 12);
    auto put = [&](unsigned x) { key += std::to_string(x); key += '.'; };
    key += "E"; put(variant.vec); put(variant.packed16); put(variant.index64); put(options.block); put(options.unroll); put(options.strictMath); put(options.rowMinBlocks);
    key += "L";
    for (size_t i = 0; i < spec.loads.size(); ++i)
    {
        const auto& l = spec.loads[i];
        Path p = loadPath(l, (variant.fastLoads >> i) & 1u);
        put(l.view.dtype); put(static_cast<unsigned>(p));
        if (p == Path::General) put(l.view.rank);
    }
    key += "N";
    for (const auto& nd : spec.nodes)
    {
        put(static_cast<unsigned>(nd.op)); put(nd.dtype); put(nd.srcDtype);
        put(nd.a.kind); put(nd.a.index); put(nd.b.kind); put(nd.b.index); put(nd.scalarIndex);
    }
    key += "S";
    for (size_t i = 0; i < spec.stores.size(); ++i)
    {
        const auto& s = spec.stores[i];
        Path p = storePath(s, (variant.fastStores >> i) & 1u);
        put(s.view.dtype); put(static_cast<unsigned>(p)); put(s.node);
        if (p == Path::General) put(s.view.rank);
    }
    if (!spec.reductions.empty())
    {
        key += "R";
        for (const auto& r : spec.reductions) { put(r.node); put(r.isMax); put(r.dtype); put(r.absBits); }
    }
    if (variant.rowMode)
    {
        key += "W"; put(variant.warpPerRow);
        for (const auto& r : spec.rowReductions) { put(r.node); put(r.isMax); put(r.dtype); put(r.initImmediate); put(r.scalarIndex); }
    }
    return key;
}

std::vector<uint64_t> packKernelArguments(const KernelSpec& spec, const KernelVariant& variant, void* scratch)
{
    std::vector<uint64_t> a;
    a.reserve(spec.loads.size() * 3 + spec.stores.size() * 3 + spec.scalars.size() + 1);
    for (auto& l : spec.loads) a.push_back(reinterpret_cast<uint64_t>(l.view.firstByte()));
    for (auto& s : spec.stores) a.push_back(reinterpret_cast<uint64_t>(s.view.firstByte()));
    a.push_back(spec.count);
    for (auto& sc : spec.scalars) a.push_back(sc.raw);
    auto pushLayout = [&](const View& v)
    {
        for (int d = 0; d < v.rank; ++d) a.push_back(v.shape[d]);
        for (int d = 0; d < v.rank; ++d) a.push_back(v.strides[d]);
    };
    for (size_t i = 0; i < spec.loads.size(); ++i)
    {
        const auto& l = spec.loads[i];
        switch (loadPath(l, (variant.fastLoads >> i) & 1u))
        {
            case Path::RowWide: a.push_back(l.view.shape[1]); break;
            case Path::ColWide: a.push_back(l.view.shape[1]); a.push_back(l.view.strides[0]); break;
            case Path::General: pushLayout(l.view); break;
            default: break;
        }
    }
    for (size_t i = 0; i < spec.stores.size(); ++i)
        if (storePath(spec.stores[i], (variant.fastStores >> i) & 1u) == Path::General) pushLayout(spec.stores[i].view);
    if (!spec.reductions.empty())
    {
        for (const auto& r : spec.reductions) a.push_back(reinterpret_cast<uint64_t>(r.out.firstByte()));
        a.push_back(reinterpret_cast<uint64_t>(scratch));
    }
    if (variant.rowMode)
    {
        a.push_back(spec.rowCols);
        for (const auto& r : spec.rowReductions) a.push_back(reinterpret_cast<uint64_t>(r.out.firstByte()));
    }
    return a;
}

std::string generateKernelSource(const KernelSpec& spec, const KernelVariant& variant, const CodegenOptions& options,
                                 const std::string& entryName)
{
    const bool tunedRows16 = variant.rowMode && variant.packed16 && options.rowMinBlocks < 0;
    const int E = variant.vec, U = tunedRows16 ? 1 : options.unroll, B = options.block;
    const int rowMinBlocks = tunedRows16 ? 8 : std::max(0, options.rowMinBlocks);
    const size_t nL = spec.loads.size(), nS = spec.stores.size();
    std::ostringstream o;
    o << "#define AIX_FAST " << (options.strictMath ? 0 : 1) << "\n" << kPrelude << "\n";
    o << "typedef " << (variant.index64 ? "unsigned long long" : "unsigned int") << " idx_t;\n";

    // ---- argument slots -------------------------------------------------------------------------------------------
    size_t slot = nL + nS;
    const size_t slotCount = slot++;
    const size_t slotScalars = slot;
    slot += spec.scalars.size();
    std::vector<size_t> loadAux(nL, 0), storeAux(nS, 0);
    std::vector<Path> lp(nL), sp(nS);
    for (size_t i = 0; i < nL; ++i)
    {
        lp[i] = loadPath(spec.loads[i], (variant.fastLoads >> i) & 1u);
        loadAux[i] = slot;
        if (lp[i] == Path::RowWide) slot += 1;
        else if (lp[i] == Path::ColWide) slot += 2;
        else if (lp[i] == Path::General) slot += 2 * spec.loads[i].view.rank;
    }
    for (size_t i = 0; i < nS; ++i)
    {
        sp[i] = storePath(spec.stores[i], (variant.fastStores >> i) & 1u);
        storeAux[i] = slot;
        if (sp[i] == Path::General) slot += 2 * spec.stores[i].view.rank;
    }
    const size_t nR = spec.reductions.size();
    const size_t slotReductions = slot;
    slot += nR;
    const size_t slotScratch = slot;
    if (nR) ++slot;
    const size_t nRR = spec.rowReductions.size();
    const size_t slotRowCols = slot;
    if (variant.rowMode) slot += 1 + nRR;
    o << "struct Params { u64_t a[" << std::max<size_t>(slot, 1) << "]; };\n\n";

    auto T = [&](uint8_t dt) { return std::string(kTraits[dt]); };
    auto arg = [&](size_t s) { return "p.a[" + std::to_string(s) + "]"; };

    // Offset (in elements) of logical element `i` inside a general strided view whose layout sits at slot `aux`.
    auto emitGeneralOffset = [&](std::ostream& os, const std::string& var, const std::string& i, int rank, size_t aux,
                                 const std::string& indent)
    {
        os << indent << "idx_t " << var << " = 0;\n";
        if (rank == 0) return;
        os << indent << "{ idx_t r_ = " << i << ";\n";
        for (int d = rank - 1; d >= 1; --d)
        {
            os << indent << "  { const idx_t e_ = (idx_t)" << arg(aux + d) << "; const idx_t q_ = r_ / e_; " << var
               << " += (r_ - q_ * e_) * (idx_t)" << arg(aux + rank + d) << "; r_ = q_; }\n";
        }
        os << indent << "  " << var << " += r_ * (idx_t)" << arg(aux + rank) << "; }\n";
    };

    // The straight-line SSA body for one element. `in(l)` yields the expression of load l's storage value.
    auto emitNodes = [&](std::ostream& os, const std::string& indent, auto&& in)
    {
        auto operand = [&](const OperandRef& r, uint8_t want) -> std::string
        {
            if (r.kind == OperandRef::Reg)
            {
                uint8_t have = spec.nodes[r.index].dtype;
                std::string v = "v" + std::to_string(r.index);
                return have == want ? v : "op_cast<" + T(have) + ", " + T(want) + ">(" + v + ")";
            }
            uint8_t have = spec.loads[r.index].view.dtype;
            std::string v = T(have) + "::ld(" + in(r.index) + ")";
            return have == want ? v : "op_cast<" + T(have) + ", " + T(want) + ">(" + v + ")";
        };
        for (size_t k = 0; k < spec.nodes.size(); ++k)
        {
            const KernelNode& nd = spec.nodes[k];
            const std::string D = T(nd.dtype);
            os << indent << "const " << D << "::C v" << k << " = ";
            switch (nd.op)
            {
                case Op::Fill:
                    os << D << "::ld(sc" << nd.scalarIndex << ")";
                    break;
                case Op::Cast:
                {
                    // operand in its own type, then converted
                    OperandRef r = nd.a;
                    uint8_t have = r.kind == OperandRef::Reg ? spec.nodes[r.index].dtype : spec.loads[r.index].view.dtype;
                    os << "op_cast<" << T(have) << ", " << D << ">(" << operand(r, have) << ")";
                    break;
                }
                case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: case Op::Pow:
                    os << "op_" << opName(nd.op) << "<" << D << ">(" << operand(nd.a, nd.dtype) << ", " << operand(nd.b, nd.dtype) << ")";
                    break;
                default:
                    os << "op_" << opName(nd.op) << "<" << D << ">(" << operand(nd.a, nd.dtype) << ")";
                    break;
            }
            os << ";\n";
        }
    };

    // Same body on register pairs (variant.packed16): every value is an `unsigned` holding two 16-bit floats.
    auto emitNodesPacked = [&](std::ostream& os, const std::string& indent, auto&& in)
    {
        auto operand = [&](const OperandRef& r) -> std::string
        {
            return r.kind == OperandRef::Reg ? "v" + std::to_string(r.index) : in(r.index);
        };
        for (size_t k = 0; k < spec.nodes.size(); ++k)
        {
            const KernelNode& nd = spec.nodes[k];
            const std::string D = T(nd.dtype);
            os << indent << "const unsigned v" << k << " = ";
            switch (nd.op)
            {
                case Op::Fill:
                    os << "P2<" << D << ">::splat(sc" << nd.scalarIndex << ")";
                    break;
                case Op::Add: case Op::Sub: case Op::Mul: case Op::Div: case Op::Pow:
                    os << "pp_" << opName(nd.op) << "<" << D << ">(" << operand(nd.a) << ", " << operand(nd.b) << ")";
                    break;
                default:
                    os << "pp_" << opName(nd.op) << "<" << D << ">(" << operand(nd.a) << ")";
                    break;
            }
            os << ";\n";
        }
    };

    o << "extern \"C\" __global__ void __launch_bounds__(" << B << ((variant.rowMode && rowMinBlocks > 0) ? ", " + std::to_string(rowMinBlocks) : std::string()) << ") " << entryName
      << "(const __grid_constant__ Params p)\n{\n";
    o << "    const idx_t n = (idx_t)" << arg(slotCount) << ";\n";
    for (size_t i = 0; i < nL; ++i)
        o << "    const " << T(spec.loads[i].view.dtype) << "::S* const l" << i << " = (const " << T(spec.loads[i].view.dtype)
          << "::S*)" << arg(i) << ";\n";
    for (size_t i = 0; i < nS; ++i)
        o << "    " << T(spec.stores[i].view.dtype) << "::S* const s" << i << " = (" << T(spec.stores[i].view.dtype)
          << "::S*)" << arg(nL + i) << ";\n";
    for (size_t i = 0; i < spec.scalars.size(); ++i)
    {
        const std::string S = T(spec.scalarDtypes[i]) + "::S";
        o << "    " << S << " sc" << i << "; { const u64_t raw_ = " << arg(slotScalars + i) << "; sc" << i << " = *(const " << S
          << "*)&raw_; }\n";
    }
    for (size_t i = 0; i < nL; ++i)
        if (lp[i] == Path::Scalar) o << "    const " << T(spec.loads[i].view.dtype) << "::S x" << i << "s = l" << i << "[0];\n";

    auto redType = [&](size_t r) { return spec.reductions[r].absBits ? std::string("RedAbsBits")
                                                                        : "Red<" + T(spec.reductions[r].dtype) + ", " + (spec.reductions[r].isMax ? "true" : "false") + ">"; };
    for (size_t r = 0; r < nR; ++r)
        o << "    " << redType(r) << "::A racc" << r << " = " << redType(r) << "::init();\n";
    auto emitReduceSteps = [&](std::ostream& os, const std::string& indent)
    {
        for (size_t r = 0; r < nR; ++r)
            os << indent << "racc" << r << " = " << redType(r) << "::step(racc" << r << ", v" << spec.reductions[r].node << ");\n";
    };

    // ---- row mode: one warp or one CTA per row of rowCols elements, per-row folds at the end of every row ------------
    if (variant.rowMode)
    {
        const bool RW = variant.warpPerRow;
        const int lanes = RW ? 32 : B;
        auto rowRedType = [&](size_t r) { return "Red<" + T(spec.rowReductions[r].dtype) + ", " + (spec.rowReductions[r].isMax ? "true" : "false") + ">"; };
        auto emitRowSteps = [&](std::ostream& os, const std::string& indent)
        {
            for (size_t r = 0; r < nRR; ++r)
                os << indent << "rr" << r << " = " << rowRedType(r) << "::step(rr" << r << ", v" << spec.rowReductions[r].node << ");\n";
        };
        o << "    const idx_t cols = (idx_t)" << arg(slotRowCols) << ";\n";
        o << "    const idx_t rows = n / cols;\n";
        o << "    const int lane = " << (RW ? "threadIdx.x & 31" : "threadIdx.x") << ";\n";
        o << "    __shared__ u64_t rsm[32];\n";
        o << "    for (idx_t row0 = (idx_t)blockIdx.x * " << (RW ? B / 32 : 1) << "; row0 < rows; row0 += (idx_t)gridDim.x * " << (RW ? B / 32 : 1) << ")\n    {\n";
        o << "        const idx_t row = row0 + " << (RW ? "(threadIdx.x >> 5)" : "0") << ";\n";
        for (size_t r = 0; r < nRR; ++r)
            o << "        " << rowRedType(r) << "::A rr" << r << " = " << rowRedType(r) << "::init();\n";
        o << "        if (row < rows)\n        {\n";
        o << "            const idx_t rowBase = row * cols;\n";
        for (size_t i = 0; i < nL; ++i)
            if (lp[i] == Path::ColWide)
                o << "            const " << T(spec.loads[i].view.dtype) << "::S xc" << i << " = l" << i << "[row * (idx_t)" << arg(loadAux[i] + 1) << "];\n";
        if (E > 1)
        {
            o << "            const idx_t cpk = cols / " << E << ";\n";
            o << "            for (idx_t cp = lane; cp < cpk; cp += " << (lanes * U) << ")\n            {\n";
            o << "                bool ok[" << U << "];\n";
            for (size_t i = 0; i < nL; ++i)
                if (lp[i] != Path::Scalar && lp[i] != Path::ColWide)
                    o << "                Pack<" << T(spec.loads[i].view.dtype) << "::S, " << E << "> x" << i << "[" << U << "];\n";
            o << "                #pragma unroll\n                for (int u = 0; u < " << U << "; ++u)\n                {\n";
            o << "                    const idx_t q = cp + (idx_t)u * " << lanes << ";\n";
            o << "                    ok[u] = q < cpk;\n";
            o << "                    if (!ok[u]) continue;\n";
            for (size_t i = 0; i < nL; ++i)
            {
                const std::string S = T(spec.loads[i].view.dtype) + "::S";
                switch (lp[i])
                {
                    case Path::DenseWide:
                        o << "                    x" << i << "[u] = *(const Pack<" << S << ", " << E << ">*)(l" << i << " + rowBase + q * " << E << ");\n";
                        break;
                    case Path::DenseElem:
                        o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e) x" << i << "[u].v[e] = l" << i << "[rowBase + q * " << E << " + e];\n";
                        break;
                    case Path::RowWide:
                        o << "                    x" << i << "[u] = *(const Pack<" << S << ", " << E << ">*)(l" << i << " + q * " << E << ");\n";
                        break;
                    case Path::General:
                        o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e)\n                    {\n";
                        emitGeneralOffset(o, "off_", "(rowBase + q * " + std::to_string(E) + " + e)", spec.loads[i].view.rank, loadAux[i], "                        ");
                        o << "                        x" << i << "[u].v[e] = l" << i << "[off_];\n                    }\n";
                        break;
                    default: break;
                }
            }
            o << "                }\n";
            o << "                #pragma unroll\n                for (int u = 0; u < " << U << "; ++u)\n                {\n";
            o << "                    if (!ok[u]) continue;\n";
            o << "                    const idx_t q = cp + (idx_t)u * " << lanes << ";\n";
            for (size_t i = 0; i < nS; ++i)
                o << "                    Pack<" << T(spec.stores[i].view.dtype) << "::S, " << E << "> y" << i << ";\n";
            if (variant.packed16)
            {
                o << "                    #pragma unroll\n                    for (int e = 0; e < " << (E / 2) << "; ++e)\n                    {\n";
                emitNodesPacked(o, "                        ", [&](size_t l) -> std::string
                {
                    const std::string P = "P2<" + T(spec.loads[l].view.dtype) + ">::";
                    if (lp[l] == Path::Scalar) return P + "splat(x" + std::to_string(l) + "s)";
                    if (lp[l] == Path::ColWide) return P + "splat(xc" + std::to_string(l) + ")";
                    return P + "join(x" + std::to_string(l) + "[u].v[2 * e], x" + std::to_string(l) + "[u].v[2 * e + 1])";
                });
                for (size_t i = 0; i < nS; ++i)
                    o << "                        y" << i << ".v[2 * e] = (u16_t)(v" << spec.stores[i].node << " & 0xffffu); y" << i
                      << ".v[2 * e + 1] = (u16_t)(v" << spec.stores[i].node << " >> 16);\n";
                for (size_t r = 0; r < nR; ++r)
                {
                    const std::string P = "P2<" + T(spec.reductions[r].dtype) + ">::", v = "v" + std::to_string(spec.reductions[r].node);
                    o << "                        racc" << r << " = " << redType(r) << "::step(" << redType(r) << "::step(racc" << r << ", " << P << "lo(" << v
                      << ")), " << P << "hi(" << v << "));\n";
                }
                for (size_t r = 0; r < nRR; ++r)
                {
                    const std::string P = "P2<" + T(spec.rowReductions[r].dtype) + ">::", v = "v" + std::to_string(spec.rowReductions[r].node);
                    o << "                        rr" << r << " = " << rowRedType(r) << "::step(" << rowRedType(r) << "::step(rr" << r << ", " << P << "lo(" << v
                      << ")), " << P << "hi(" << v << "));\n";
                }
                o << "                    }\n";
            }
            else
            {
                o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e)\n                    {\n";
                emitNodes(o, "                        ", [&](size_t l) -> std::string
                {
                    if (lp[l] == Path::Scalar) return "x" + std::to_string(l) + "s";
                    if (lp[l] == Path::ColWide) return "xc" + std::to_string(l);
                    return "x" + std::to_string(l) + "[u].v[e]";
                });
                for (size_t i = 0; i < nS; ++i)
                    o << "                        y" << i << ".v[e] = " << T(spec.stores[i].view.dtype) << "::st(" << "v" << spec.stores[i].node << ");\n";
                emitReduceSteps(o, "                        ");
                emitRowSteps(o, "                        ");
                o << "                    }\n";
            }
            for (size_t i = 0; i < nS; ++i)
            {
                const std::string S = T(spec.stores[i].view.dtype) + "::S";
                if (sp[i] == Path::DenseWide)
                    o << "                    *(Pack<" << S << ", " << E << ">*)(s" << i << " + rowBase + q * " << E << ") = y" << i << ";\n";
                else if (sp[i] == Path::DenseElem)
                    o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e) s" << i << "[rowBase + q * " << E << " + e] = y" << i << ".v[e];\n";
                else
                {
                    o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e)\n                    {\n";
                    emitGeneralOffset(o, "off_", "(rowBase + q * " + std::to_string(E) + " + e)", spec.stores[i].view.rank, storeAux[i], "                        ");
                    o << "                        s" << i << "[off_] = y" << i << ".v[e];\n                    }\n";
                }
            }
            o << "                }\n            }\n";
        }
        else
        {
            o << "            for (idx_t c = lane; c < cols; c += " << lanes << ")\n            {\n";
            o << "                const idx_t i = rowBase + c;\n";
            for (size_t l = 0; l < nL; ++l)
            {
                const View& v = spec.loads[l].view;
                const std::string S = T(v.dtype) + "::S";
                switch (lp[l])
                {
                    case Path::Scalar: case Path::ColWide: break;
                    case Path::DenseWide: case Path::DenseElem:
                        o << "                const " << S << " t" << l << " = l" << l << "[i];\n";
                        break;
                    case Path::RowWide:
                        o << "                const " << S << " t" << l << " = l" << l << "[c];\n";
                        break;
                    case Path::General:
                        emitGeneralOffset(o, "off" + std::to_string(l), "i", v.rank, loadAux[l], "                ");
                        o << "                const " << S << " t" << l << " = l" << l << "[off" << l << "];\n";
                        break;
                }
            }
            emitNodes(o, "                ", [&](size_t l) -> std::string
            {
                if (lp[l] == Path::Scalar) return "x" + std::to_string(l) + "s";
                if (lp[l] == Path::ColWide) return "xc" + std::to_string(l);
                return "t" + std::to_string(l);
            });
            for (size_t i = 0; i < nS; ++i)
            {
                const std::string D = T(spec.stores[i].view.dtype);
                if (sp[i] == Path::General)
                {
                    emitGeneralOffset(o, "so" + std::to_string(i), "i", spec.stores[i].view.rank, storeAux[i], "                ");
                    o << "                s" << i << "[so" << i << "] = " << D << "::st(v" << spec.stores[i].node << ");\n";
                }
                else
                    o << "                s" << i << "[i] = " << D << "::st(v" << spec.stores[i].node << ");\n";
            }
            emitReduceSteps(o, "                ");
            emitRowSteps(o, "                ");
            o << "            }\n";
        }
        o << "        }\n";
        // per-row folds: every thread of the block takes part (the CTA-wide fold synchronises the block)
        for (size_t r = 0; r < nRR; ++r)
        {
            const KernelRowReduce& rr = spec.rowReductions[r];
            const std::string S = T(rr.dtype) + "::S";
            o << "        {\n            const " << rowRedType(r) << "::W w_ = row_fold<" << rowRedType(r) << ", " << (RW ? "true" : "false") << ">(rr" << r << ", rsm);\n";
            o << "            if (lane == 0 && row < rows)\n            {\n";
            o << "                " << S << "* const o_ = (" << S << "*)" << arg(slotRowCols + 1 + r) << " + row;\n";
            o << "                o_[0] = " << rowRedType(r) << "::finish(" << rowRedType(r) << "::merge(" << rowRedType(r) << "::lift("
              << (rr.initImmediate ? "sc" + std::to_string(rr.scalarIndex) : std::string("o_[0]")) << "), w_));\n";
            o << "            }\n        }\n";
        }
        o << "    }\n";
        for (size_t r = 0; r < nR; ++r)
            o << "    red_finish<" << redType(r) << " >(racc" << r << ", (u64_t*)(" << arg(slotScratch) << " + " << kReductionPartialsOffset
              << "ull + " << (r * kReductionMaxBlocks * 8) << "ull), (unsigned*)(" << arg(slotScratch) << " + " << (4 * (r + 1)) << "ull), ("
              << redType(r) << "::S*)" << arg(slotReductions + r) << ");\n";
        o << "}\n";
        return o.str();
    }

    // ---- main loop: U packs of E elements per thread and iteration ----------------------------------------------
    if (E > 1)
    {
        o << "    const idx_t nvec = n / " << E << ";\n";
        o << "    if (nvec != 0)\n    {\n";
        o << "        idx_t pk = (idx_t)blockIdx.x * " << (B * U) << " + threadIdx.x;\n";
        o << "        const idx_t gstep = (idx_t)gridDim.x * " << (B * U) << ";\n";
        // hoisted broadcast state
        for (size_t i = 0; i < nL; ++i)
        {
            if (lp[i] == Path::RowWide)
            {
                o << "        const idx_t cp" << i << " = (idx_t)" << arg(loadAux[i]) << " / " << E << ";          // packs per row\n";
                o << "        idx_t c" << i << " = pk % cp" << i << ";\n";
                o << "        const idx_t ct" << i << " = (idx_t)" << B << " % cp" << i << ", cg" << i << " = (gstep - " << (B * U) << ") % cp" << i << ";\n";
            }
            else if (lp[i] == Path::ColWide)
            {
                o << "        const idx_t cp" << i << " = (idx_t)" << arg(loadAux[i]) << " / " << E << ";\n";
                o << "        idx_t r" << i << " = pk / cp" << i << ", c" << i << " = pk - r" << i << " * cp" << i << ";\n";
                o << "        const idx_t qt" << i << " = (idx_t)" << B << " / cp" << i << ", ct" << i << " = (idx_t)" << B << " - qt" << i << " * cp" << i << ";\n";
                o << "        const idx_t qg" << i << " = (gstep - " << (B * U) << ") / cp" << i << ", cg" << i << " = (gstep - " << (B * U) << ") - qg" << i << " * cp" << i << ";\n";
            }
        }
        o << "        for (; pk < nvec; pk += gstep)\n        {\n";
        o << "            bool ok[" << U << "];\n";
        for (size_t i = 0; i < nL; ++i)
        {
            const std::string S = T(spec.loads[i].view.dtype) + "::S";
            if (lp[i] == Path::Scalar) continue;
            if (lp[i] == Path::ColWide) o << "            " << S << " x" << i << "[" << U << "];\n";
            else o << "            Pack<" << S << ", " << E << "> x" << i << "[" << U << "];\n";
        }
        o << "            #pragma unroll\n            for (int u = 0; u < " << U << "; ++u)\n            {\n";
        o << "                const idx_t q = pk + (idx_t)u * " << B << ";\n";
        o << "                ok[u] = q < nvec;\n";
        o << "                if (ok[u])\n                {\n";
        for (size_t i = 0; i < nL; ++i)
        {
            const std::string S = T(spec.loads[i].view.dtype) + "::S";
            switch (lp[i])
            {
                case Path::DenseWide:
                    o << "                    x" << i << "[u] = *(const Pack<" << S << ", " << E << ">*)(l" << i << " + q * " << E << ");\n";
                    break;
                case Path::DenseElem:
                    o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e) x" << i << "[u].v[e] = l" << i << "[q * " << E << " + e];\n";
                    break;
                case Path::RowWide:
                    o << "                    x" << i << "[u] = *(const Pack<" << S << ", " << E << ">*)(l" << i << " + c" << i << " * " << E << ");\n";
                    break;
                case Path::ColWide:
                    o << "                    x" << i << "[u] = l" << i << "[r" << i << " * (idx_t)" << arg(loadAux[i] + 1) << "];\n";
                    break;
                case Path::General:
                    o << "                    #pragma unroll\n                    for (int e = 0; e < " << E << "; ++e)\n                    {\n";
                    emitGeneralOffset(o, "off_", "(q * " + std::to_string(E) + " + e)", spec.loads[i].view.rank, loadAux[i], "                        ");
                    o << "                        x" << i << "[u].v[e] = l" << i << "[off_];\n                    }\n";
                    break;
                default: break;
            }
        }
        o << "                }\n";
        for (size_t i = 0; i < nL; ++i)
        {
            if (lp[i] == Path::RowWide)
                o << "                c" << i << " += ct" << i << "; if (c" << i << " >= cp" << i << ") c" << i << " -= cp" << i << ";\n";
            else if (lp[i] == Path::ColWide)
                o << "                r" << i << " += qt" << i << "; c" << i << " += ct" << i << "; if (c" << i << " >= cp" << i << ") { c" << i << " -= cp" << i << "; ++r" << i << "; }\n";
        }
        o << "            }\n";
        for (size_t i = 0; i < nL; ++i)
        {
            if (lp[i] == Path::RowWide)
                o << "            c" << i << " += cg" << i << "; if (c" << i << " >= cp" << i << ") c" << i << " -= cp" << i << ";\n";
            else if (lp[i] == Path::ColWide)
                o << "            r" << i << " += qg" << i << "; c" << i << " += cg" << i << "; if (c" << i << " >= cp" << i << ") { c" << i << " -= cp" << i << "; ++r" << i << "; }\n";
        }
        o << "            #pragma unroll\n            for (int u = 0; u < " << U << "; ++u)\n            {\n";
        o << "                if (!ok[u]) continue;\n";
        o << "                const idx_t q = pk + (idx_t)u * " << B << ";\n";
        for (size_t i = 0; i < nS; ++i)
            o << "                Pack<" << T(spec.stores[i].view.dtype) << "::S, " << E << "> y" << i << ";\n";
        if (variant.packed16)
        {
            o << "                #pragma unroll\n                for (int e = 0; e < " << (E / 2) << "; ++e)\n                {\n";
            emitNodesPacked(o, "                    ", [&](size_t l) -> std::string
            {
                const std::string P = "P2<" + T(spec.loads[l].view.dtype) + ">::";
                if (lp[l] == Path::Scalar) return P + "splat(x" + std::to_string(l) + "s)";
                if (lp[l] == Path::ColWide) return P + "splat(x" + std::to_string(l) + "[u])";
                return P + "join(x" + std::to_string(l) + "[u].v[2 * e], x" + std::to_string(l) + "[u].v[2 * e + 1])";
            });
            for (size_t i = 0; i < nS; ++i)
                o << "                    y" << i << ".v[2 * e] = (u16_t)(v" << spec.stores[i].node << " & 0xffffu); y" << i
                  << ".v[2 * e + 1] = (u16_t)(v" << spec.stores[i].node << " >> 16);\n";
            // reductions fold both halves of the packed register, widened to float
            for (size_t r = 0; r < nR; ++r)
            {
                const std::string P = "P2<" + T(spec.reductions[r].dtype) + ">::", v = "v" + std::to_string(spec.reductions[r].node);
                o << "                    racc" << r << " = " << redType(r) << "::step(" << redType(r) << "::step(racc" << r << ", " << P << "lo(" << v
                  << ")), " << P << "hi(" << v << "));\n";
            }
            o << "                }\n";
        }
        else
        {
        o << "                #pragma unroll\n                for (int e = 0; e < " << E << "; ++e)\n                {\n";
        emitNodes(o, "                    ", [&](size_t l) -> std::string
        {
            if (lp[l] == Path::Scalar) return "x" + std::to_string(l) + "s";
            if (lp[l] == Path::ColWide) return "x" + std::to_string(l) + "[u]";
            return "x" + std::to_string(l) + "[u].v[e]";
        });
        for (size_t i = 0; i < nS; ++i)
            o << "                    y" << i << ".v[e] = " << T(spec.stores[i].view.dtype) << "::st(" << "v" << spec.stores[i].node << ");\n";
        emitReduceSteps(o, "                    ");
        o << "                }\n";
        }
        for (size_t i = 0; i < nS; ++i)
        {
            const std::string S = T(spec.stores[i].view.dtype) + "::S";
            if (sp[i] == Path::DenseWide)
                o << "                *(Pack<" << S << ", " << E << ">*)(s" << i << " + q * " << E << ") = y" << i << ";\n";
            else if (sp[i] == Path::DenseElem)
                o << "                #pragma unroll\n                for (int e = 0; e < " << E << "; ++e) s" << i << "[q * " << E << " + e] = y" << i << ".v[e];\n";
            else
            {
                o << "                #pragma unroll\n                for (int e = 0; e < " << E << "; ++e)\n                {\n";
                emitGeneralOffset(o, "off_", "(q * " + std::to_string(E) + " + e)", spec.stores[i].view.rank, storeAux[i], "                    ");
                o << "                    s" << i << "[off_] = y" << i << ".v[e];\n                }\n";
            }
        }
        o << "            }\n        }\n    }\n";
    }

    // ---- tail (or the whole tensor when E == 1): one element per thread -----------------------------------------
    if (E > 1) o << "    const idx_t tail0 = nvec * " << E << ";\n";
    else       o << "    const idx_t tail0 = 0;\n";
    o << "    for (idx_t i = tail0 + (idx_t)blockIdx.x * " << B << " + threadIdx.x; i < n; i += (idx_t)gridDim.x * " << B << ")\n    {\n";
    for (size_t l = 0; l < nL; ++l)
    {
        const View& v = spec.loads[l].view;
        const std::string S = T(v.dtype) + "::S";
        switch (lp[l])
        {
            case Path::Scalar: break;
            case Path::DenseWide: case Path::DenseElem:
                o << "        const " << S << " t" << l << " = l" << l << "[i];\n";
                break;
            case Path::RowWide:
                o << "        const " << S << " t" << l << " = l" << l << "[i % (idx_t)" << arg(loadAux[l]) << "];\n";
                break;
            case Path::ColWide:
                o << "        const " << S << " t" << l << " = l" << l << "[(i / (idx_t)" << arg(loadAux[l]) << ") * (idx_t)" << arg(loadAux[l] + 1) << "];\n";
                break;
            case Path::General:
                emitGeneralOffset(o, "off" + std::to_string(l), "i", v.rank, loadAux[l], "        ");
                o << "        const " << S << " t" << l << " = l" << l << "[off" << l << "];\n";
                break;
        }
    }
    emitNodes(o, "        ", [&](size_t l) -> std::string
    {
        return lp[l] == Path::Scalar ? "x" + std::to_string(l) + "s" : "t" + std::to_string(l);
    });
    for (size_t i = 0; i < nS; ++i)
    {
        const std::string D = T(spec.stores[i].view.dtype);
        if (sp[i] == Path::General)
        {
            emitGeneralOffset(o, "so" + std::to_string(i), "i", spec.stores[i].view.rank, storeAux[i], "        ");
            o << "        s" << i << "[so" << i << "] = " << D << "::st(v" << spec.stores[i].node << ");\n";
        }
        else
            o << "        s" << i << "[i] = " << D << "::st(v" << spec.stores[i].node << ");\n";
    }
    emitReduceSteps(o, "        ");
    o << "    }\n";
    // ---- reduction epilogue: every thread of every block arrives here ------------------------------------------------
    for (size_t r = 0; r < nR; ++r)
        o << "    red_finish<" << redType(r) << " >(racc" << r << ", (u64_t*)(" << arg(slotScratch) << " + " << kReductionPartialsOffset
          << "ull + " << (r * kReductionMaxBlocks * 8) << "ull), (unsigned*)(" << arg(slotScratch) << " + " << (4 * (r + 1)) << "ull), ("
          << redType(r) << "::S*)" << arg(slotReductions + r) << ");\n";
    o << "}\n";
    return o.str();
}

}   // namespace aixb200
