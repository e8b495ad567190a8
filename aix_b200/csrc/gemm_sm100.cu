// Dense matmul on the 5th-generation tensor cores of sm_100a.
//
// Replaces the reference's threadgroup-tiled Metal GEMM (matrixMulStridedTiled<16>, aixDeviceMetalShaders.hpp:1191-1275,
// selected in aixDeviceMetal.cpp:569-656). Two kernels share one structure:
//   * persistent CTAs (one per SM) walk the output tiles in an L2-friendly order;
//   * warp 0 streams operand tiles with TMA (cp.async.bulk.tensor, no multicast) into a ring of 128-byte-swizzled
//     shared-memory stages, signalling mbarriers;
//   * warp 1 issues tcgen05.mma from one elected thread; the accumulators live in tensor memory (TMEM), two buffers of
//     256 columns so that the epilogue of one tile overlaps the main loop of the next; tcgen05.commit releases
//     shared-memory stages and publishes finished accumulators;
//   * warps 2-5 read the accumulator with tcgen05.ld, convert and write C.
// gemmPairKernel (the default): clusters of two CTAs compute 256 x 256 tiles with cta_group::2 - each CTA loads its own
// 128 rows of A and half of the B tile, the leader issues M=256 MMAs for both SMs; 3 stages of two swizzle atoms along K
// (one 3-D TMA box per operand and stage); C leaves through shared memory and TMA stores. gemmKernel: one CTA per
// 128 x 256 tile, 4 stages of one atom, row-per-thread epilogue; used for M <= 128 and as a cross-check.
// Operands may be K-major or MN-major (row- or column-major views): the shared-memory matrix descriptors and the
// TMA boxes are chosen per operand, so forward (A.B), dX (G.B^T) and dW (A^T.G) run without materialised transposes.
// f32 problems run on the 16-bit pipes from split operands (pair kernel: two fp16 terms per scaled operand, three
// passes, in an instantiation of its own whose issue loops do not depend on the pass; single-CTA kernel and the
// AIXB200_GEMM_F32=hybrid form: a TF32 main pass plus two bf16 cross-term passes). Because the tensor core's f32
// accumulation truncates, K is cut into chunks whose partial sums are added with IEEE additions: in the three-pass
// kernel in registers of eight epilogue warps (C is stored once per tile), in the hybrid form by TMA reduce-add in L2 or
// by the epilogue threads on the direct path. A tensor's two-term form is prepared once and cached by the device
// (Device::PreparedTerms); it is read K-major or MN-major, whichever the view asks for.
// Every wait on an mbarrier or on a flag of another cluster is bounded in time; on expiry the kernel raises an error
// word and drains.
#include "gemm.hpp"

#include "device.hpp"
#include "dtypes.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <mutex>

namespace aixb200::gemm
{

namespace
{

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kStageBytesA = kBlockM * 128;              // 128 rows (or 2 MN atoms x 64 k) x 128 B
constexpr int kStageBytesB = kBlockN * 128;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kThreadsHalfTerms = 320;                   // three-fp16-pass f32 kernel: eight epilogue warps (see its epilogue)
constexpr int kTmemColumns = 512;
constexpr uint64_t kWaitLimitNs = 2000000000ull;         // 2 s: far beyond any legitimate wait

struct KernelParams
{
    uint32_t m, n, k;
    uint32_t tilesM, tilesN, kBlocks;
    uint32_t tileGroup;         // row-tiles walked together (tile order)
    uint32_t blockK;            // elements of K per stage (64 for 16-bit, 32 for tf32)
    uint32_t blockN;            // output tile width: 256, or 128 when that fills the last wave of tiles better
    uint32_t aMnMajor, bMnMajor;
    uint32_t aBoxes, bBoxes;    // TMA boxes per stage and operand
    uint32_t aBoxBytes, bBoxBytes;
    uint32_t aBoxStepMn, bBoxStepMn;   // MN elements covered by one box (MN-major) / unused (K-major)
    // pair kernel (stages of two swizzle atoms along K):
    uint32_t aLoad3d, bLoad3d;  // the operand's stage is ONE box of a 3-D map, else 2-D boxes of one atom each
    uint32_t pairABytes, pairBBytes;   // bytes per stage and CTA
    uint32_t pairAOff[8], pairBOff[8]; // shared-memory descriptor start of the stage's 8 MMAs, in 16-byte units
    uint32_t pairALbo, pairBLbo;
    uint32_t atomK;             // K elements per swizzle atom in the main pass: 64 (16-bit) or 32 (TF32); cross passes: 64
    uint32_t halfTerms;         // f32 problems as three fp16 passes over scaled two-term operands (see splitF16Kernel)
    const uint32_t* scaleA;     // halfTerms: bit pattern of max|A| (device memory), for the output scale
    const uint32_t* scaleB;     //            and of max|B|
    uint32_t aPlane, bPlane;    // distance in elements from an operand's first term (or `hi` part) to its second: along K for a
                                // K-major operand, along M / N for an MN-major one
    uint32_t idesc;             // tcgen05 instruction descriptor
    uint32_t idesc16;           // f32 problems: descriptor of the bf16 cross-term passes
    uint32_t aLbo, bLbo;        // leading byte offsets (MN-major), 0 for K-major
    uint32_t kAdvanceA, kAdvanceB;     // bytes to advance the descriptor start per MMA along K
    uint32_t mmasPerStage;
    uint32_t outDtype;          // F32, F16, BF16
    uint32_t kPhases;           // 1, or 3 for f32 problems: two bf16 cross-term passes, then the TF32 main pass
    uint32_t kPerPhase;         // f32 problems: padded K = offset of the `lo` half inside the bf16 split buffers
    uint32_t chunkBlocks;       // k-blocks folded inside TMEM before the partial result is added to C in f32
    uint32_t chunks;            // number of such partial results per tile (1: plain store)
    uint32_t vectorStores;      // C rows are 16-byte aligned
    uint32_t tmaEpilogue;       // pair kernel: C leaves through shared memory and TMA stores / f32 reduce-adds
    uint32_t splitTiles;        // pair kernel: tiles [0, splitTiles) are cut along K and shared by all clusters
    uint32_t splitUnits;        // splitTiles * kBlocks
    void*    c;
    uint32_t* errorWord;
    float*   splitWorkspace;    // one 256 x 256 f32 partial accumulator per cluster
    uint32_t* splitCounters;    // per (split tile, CTA rank): partial accumulators published so far; left at zero
    // Tiles handed out at run time (see WorkIterator): null = the static deal
    uint32_t* tileCounters;     // eight counters, 16 words apart; launch e uses counter e % 8 and zeroes counter (e + 4) % 8
    uint64_t* tileRing;         // per cluster kGemmRingSlots entries: (epoch << 40) | (iteration << 20) | tile
    uint32_t tileEpoch;         // launch number on this device, 24 bits
    // Elementwise consumers folded into the epilogue of the three-fp16-pass f32 kernel (see Problem::bias):
    uint32_t outputs;           // bit 0: C itself, bit 1: C + bias (through mapC1), bit 2: tanh(C + bias) (through mapC2)
    const float* bias;          // n values, added to every row
    uint32_t* maxSlot;          // max|x| of the last output as a bit pattern (atomic maximum; zeroed before the launch), or null
};

// ---- PTX wrappers ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarExpectTx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTest(uint64_t* bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(smemAddr(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t globalTimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: returns false (and raises *abortFlag) when the barrier did not flip within kWaitLimitNs or when
// another role already gave up.
__device__ __forceinline__ bool mbarWait(uint64_t* bar, uint32_t parity, volatile uint32_t* abortFlag, uint64_t limitNs = kWaitLimitNs)
{
    if (mbarTest(bar, parity)) return true;
    const uint64_t start = globalTimerNs();
    uint32_t spins = 0;
    while (!mbarTest(bar, parity))
    {
        if ((++spins & 63u) == 0)
        {
            if (*abortFlag) return false;
            if (globalTimerNs() - start > limitNs) { *abortFlag = 1; return false; }
        }
    }
    return true;
}
// After a wait has run out, the thread that issued TMA copies lingers for a bounded time before the CTA gives its
// shared memory back, so that copies still in flight land in memory this CTA still owns.
__device__ __forceinline__ void lingerAfterAbort(volatile uint32_t* abortFlag)
{
    if (!*abortFlag) return;
    const uint64_t start = globalTimerNs();
    while (globalTimerNs() - start < 1000000ull) { }          // 1 ms: orders of magnitude above a copy's latency
}
__device__ __forceinline__ void tmaLoad2d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smemAddr(dst)), "l"(map), "r"(smemAddr(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmemAlloc(uint32_t* resultInSmem, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(resultInSmem)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void fenceBeforeSync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fenceAfterSync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
template <bool Tf32>
__device__ __forceinline__ void umma(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    if (Tf32)
        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                     ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                     ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ummaCommit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void tmemLoad32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmemLoad16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte units,
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smemDescriptor(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;       // SWIZZLE_128B
    return d;
}

struct SharedStorage
{
    alignas(1024) uint8_t a[kStages][kStageBytesA];
    alignas(1024) uint8_t b[kStages][kStageBytesB];
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmemFull[2];
    uint64_t tmemEmpty[2];
    uint32_t tmemBase;
    uint32_t abortFlag;
};

__device__ __forceinline__ void tileCoordinates(uint32_t t, uint32_t tilesM, uint32_t tilesN, uint32_t kGroup, uint32_t& tm, uint32_t& tn)
{
    // kGroup row-tiles share their B columns back to back: a wave of tiles then covers a roughly square patch of C
    const uint32_t perGroup = kGroup * tilesN;
    const uint32_t group = t / perGroup;
    const uint32_t firstM = group * kGroup;
    const uint32_t groupRows = min(tilesM - firstM, kGroup);
    const uint32_t local = t - group * perGroup;
    tm = firstM + local % groupRows;
    tn = local / groupRows;
}

// Half-term scheme: an operand is multiplied by the power of two that brings its largest magnitude into [2^14, 2^15)
// before it is cut into fp16 terms. `maxBits` is the bit pattern of max|x|. Zero, infinite or NaN maxima leave the
// operand unscaled.
__device__ __forceinline__ uint32_t halfTermScaleExponent(uint32_t maxBits)
{
    const uint32_t e = (maxBits >> 23) & 0xFFu;
    if (e == 0u || e == 255u) return 127u;
    const int32_t biased = 127 + 14 - (static_cast<int32_t>(e) - 127);
    return static_cast<uint32_t>(min(max(biased, 1), 253));      // 253: the reciprocal 2^(127 - biased) stays a normal number
}
__device__ __forceinline__ float halfTermScale(uint32_t maxBits) { return __uint_as_float(halfTermScaleExponent(maxBits) << 23); }
__device__ __forceinline__ float halfTermInverseScale(uint32_t maxBits)
{
    return __uint_as_float((254u - halfTermScaleExponent(maxBits)) << 23);       // exact reciprocal: exponents 1 ... 253 map onto 253 ... 1
}

// Epilogue of one 32-column strip of one accumulator row: convert and store (first chunk) or add to what C already
// holds (later chunks of the split-f32 scheme; `old` was fetched before the TMEM load).
__device__ __forceinline__ void storeAccumulatorRow(const KernelParams& p, const uint32_t (&r)[32], const float4 (&old)[8], uint32_t row, uint32_t col, uint32_t c)
{
    if (row < p.m && col < p.n)
    {
        const bool fullRow = col + 32 <= p.n;
        if (p.outDtype == F32)
        {
            float* out = static_cast<float*>(p.c) + static_cast<size_t>(row) * p.n + col;
            // half-term scheme: undo the operands' scaling (two factors, one after the other; 1 when the scheme is off)
            const float scaleA = p.halfTerms ? halfTermInverseScale(*p.scaleA) : 1.0f;
            const float scaleB = p.halfTerms ? halfTermInverseScale(*p.scaleB) : 1.0f;
            // Partial results after the first are added to C with IEEE f32 additions: the tensor core's own
            // accumulation truncates, and that bias grows with the number of MMAs folded into one accumulator.
            if (fullRow && p.vectorStores)
            {
                #pragma unroll
                for (int v = 0; v < 8; ++v)
                {
                    float4 x = make_float4(__uint_as_float(r[4 * v]) * scaleA * scaleB, __uint_as_float(r[4 * v + 1]) * scaleA * scaleB,
                                           __uint_as_float(r[4 * v + 2]) * scaleA * scaleB, __uint_as_float(r[4 * v + 3]) * scaleA * scaleB);
                    if (c > 0) { x.x += old[v].x; x.y += old[v].y; x.z += old[v].z; x.w += old[v].w; }
                    reinterpret_cast<float4*>(out)[v] = x;
                }
            }
            else
            {
                for (uint32_t e = 0; e < 32 && col + e < p.n; ++e) out[e] = __uint_as_float(r[e]) * scaleA * scaleB + (c > 0 ? out[e] : 0.f);
            }
        }
        else
        {
            uint16_t* out = static_cast<uint16_t*>(p.c) + static_cast<size_t>(row) * p.n + col;
            uint32_t packed[16];
            #pragma unroll
            for (int v = 0; v < 16; ++v)
            {
                const float lo = __uint_as_float(r[2 * v]), hi = __uint_as_float(r[2 * v + 1]);
                const uint32_t l16 = p.outDtype == BF16 ? dev::f32ToBf16(lo) : dev::f32ToF16(lo);
                const uint32_t h16 = p.outDtype == BF16 ? dev::f32ToBf16(hi) : dev::f32ToF16(hi);
                packed[v] = l16 | (h16 << 16);
            }
            if (fullRow && p.vectorStores)
            {
                #pragma unroll
                for (int v = 0; v < 4; ++v)
                    reinterpret_cast<uint4*>(out)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
            }
            else
            {
                for (uint32_t e = 0; e < 32 && col + e < p.n; ++e)
                    out[e] = static_cast<uint16_t>((packed[e >> 1] >> ((e & 1) * 16)) & 0xFFFFu);
            }
        }
    }
}

// Epilogue of one accumulator (blockN columns of one tile row per thread). Two 32-column strips are in flight at a
// time: both TMEM loads are issued before the single wait, and for partial results after the first (split-f32 scheme)
// the values C already holds are fetched one strip pair ahead, so that neither the TMEM latency nor the global-load
// latency is paid once per strip.
__device__ __forceinline__ void loadOld(const KernelParams& p, float4 (&old)[8], uint32_t row, uint32_t col, bool wanted)
{
    if (wanted && row < p.m && col + 32 <= p.n)
    {
        const float4* in = reinterpret_cast<const float4*>(static_cast<const float*>(p.c) + static_cast<size_t>(row) * p.n + col);
        #pragma unroll
        for (int v = 0; v < 8; ++v) old[v] = in[v];
    }
}

__device__ __forceinline__ void drainAccumulator(const KernelParams& p, uint32_t taddr, uint32_t row, uint32_t colBase, uint32_t c)
{
    const bool addToC = c > 0 && p.outDtype == F32 && p.vectorStores != 0;
    float4 old0[8], old1[8];
    loadOld(p, old0, row, colBase, addToC);
    loadOld(p, old1, row, colBase + 32, addToC);
    #pragma unroll 1
    for (uint32_t c0 = 0; c0 < p.blockN; c0 += 64)
    {
        uint32_t r0[32], r1[32];
        tmemLoad32(taddr + c0, r0);
        tmemLoad32(taddr + c0 + 32, r1);
        tmemLoadWait();
        storeAccumulatorRow(p, r0, old0, row, colBase + c0, c);
        if (c0 + 64 < p.blockN) loadOld(p, old0, row, colBase + c0 + 64, addToC);
        storeAccumulatorRow(p, r1, old1, row, colBase + c0 + 32, c);
        if (c0 + 64 < p.blockN) loadOld(p, old1, row, colBase + c0 + 96, addToC);
    }
}

template <bool Tf32>
__global__ void __launch_bounds__(kThreads, 1) gemmKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                           const __grid_constant__ CUtensorMap mapA16, const __grid_constant__ CUtensorMap mapB16,
                                                           const __grid_constant__ KernelParams p)
{
    extern __shared__ uint8_t rawSmem[];
    SharedStorage& s = *reinterpret_cast<SharedStorage*>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile uint32_t* abortFlag = &s.abortFlag;

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < kStages; ++i) { mbarInit(&s.full[i], 1); mbarInit(&s.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbarInit(&s.tmemFull[i], 1); mbarInit(&s.tmemEmpty[i], 128); }
        s.abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1)
    {
        tmemAlloc(&s.tmemBase, kTmemColumns);
        tmemRelinquish();
    }
    fenceBeforeSync();
    __syncthreads();
    fenceAfterSync();
    const uint32_t tmemBase = s.tmemBase;
    const uint32_t totalTiles = p.tilesM * p.tilesN;

    if (warp == 0)
    {
        if (lane == 0)
        {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint32_t stageBytes = p.aBoxes * p.aBoxBytes + p.bBoxes * p.bBoxBytes;
            for (uint32_t t = blockIdx.x; t < totalTiles && ok; t += gridDim.x)
            {
                uint32_t tm, tn;
                tileCoordinates(t, p.tilesM, p.tilesN, p.tileGroup, tm, tn);
                const int32_t m0 = static_cast<int32_t>(tm * kBlockM), n0 = static_cast<int32_t>(tn * p.blockN);
                for (uint32_t c = 0; c < p.chunks && ok; ++c)
                {
                const uint32_t kbBegin = c * p.chunkBlocks, kbCount = min(p.kBlocks - kbBegin, p.chunkBlocks);
                for (uint32_t passIndex = 0; passIndex < p.kPhases && ok; ++passIndex)
                {
                // f32 problems: passes 0 and 1 are the cross terms lo(A).hi(B) and hi(A).lo(B) from the bf16 split
                // buffers (64 elements of K per stage); they go first, while the accumulator is still tiny. Pass 2 is
                // hi(A).hi(B) in TF32 (32 elements per stage).
                const bool cross = Tf32 && passIndex < 2;
                const uint32_t first = cross ? kbBegin >> 1 : kbBegin, count = cross ? kbCount >> 1 : kbCount;
                const uint32_t blockK = cross ? 64u : p.blockK;
                const CUtensorMap* ma = cross ? &mapA16 : &mapA;
                const CUtensorMap* mb = cross ? &mapB16 : &mapB;
                const uint32_t offA = (cross && passIndex == 0) ? p.kPerPhase : 0u, offB = (cross && passIndex == 1) ? p.kPerPhase : 0u;
                for (uint32_t kb = first; kb < first + count; ++kb)
                {
                    if (!mbarWait(&s.empty[stage], phase ^ 1u, abortFlag)) { ok = false; break; }
                    mbarExpectTx(&s.full[stage], stageBytes);
                    const int32_t kA = static_cast<int32_t>(kb * blockK + offA), kB = static_cast<int32_t>(kb * blockK + offB);
                    for (uint32_t bx = 0; bx < p.aBoxes; ++bx)
                    {
                        if (p.aMnMajor) tmaLoad2d(&s.a[stage][bx * p.aBoxBytes], ma, &s.full[stage], m0 + static_cast<int32_t>(bx * p.aBoxStepMn), kA);
                        else            tmaLoad2d(&s.a[stage][bx * p.aBoxBytes], ma, &s.full[stage], kA, m0);
                    }
                    for (uint32_t bx = 0; bx < p.bBoxes; ++bx)
                    {
                        if (p.bMnMajor) tmaLoad2d(&s.b[stage][bx * p.bBoxBytes], mb, &s.full[stage], n0 + static_cast<int32_t>(bx * p.bBoxStepMn), kB);
                        else            tmaLoad2d(&s.b[stage][bx * p.bBoxBytes], mb, &s.full[stage], kB, n0);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                }
                }
            }
        }
    }
    else if (warp == 1)
    {
        if (lane == 0)
        {
            // Descriptor halves that never change: the high word (stride offsets, version, swizzle) and the low word of
            // stage 0; per stage and per MMA only a 32-bit add remains.
            const uint64_t descHiA = smemDescriptor(0, p.aLbo, 1024), descHiB = smemDescriptor(0, p.bLbo, 1024);
            const uint32_t descLoA = (smemAddr(&s.a[0][0]) & 0x3FFFFu) >> 4, descLoB = (smemAddr(&s.b[0][0]) & 0x3FFFFu) >> 4;
            const uint32_t aStageBytes = sizeof(s.a[0]), bStageBytes = sizeof(s.b[0]);
            const uint32_t advA = p.kAdvanceA >> 4, advB = p.kAdvanceB >> 4, idesc = p.idesc, idesc16 = p.idesc16;
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < totalTiles && ok; t += gridDim.x)
            for (uint32_t c = 0; c < p.chunks && ok; ++c)
            {
                if (!mbarWait(&s.tmemEmpty[acc], accPhase ^ 1u, abortFlag)) { ok = false; break; }
                fenceAfterSync();
                const uint32_t tmemD = tmemBase + acc * kBlockN;
                const uint32_t kbCount = min(p.kBlocks - c * p.chunkBlocks, p.chunkBlocks);
                // f32 problems: kbCount bf16 stages (two cross-term passes of kbCount / 2), then kbCount TF32 stages
                const uint32_t stagesInChunk = Tf32 ? 2 * kbCount : kbCount;
                for (uint32_t it = 0; it < stagesInChunk; ++it)
                {
                    if (!mbarWait(&s.full[stage], phase, abortFlag)) { ok = false; break; }
                    fenceAfterSync();
                    const uint32_t aLo = descLoA + stage * (aStageBytes >> 4), bLo = descLoB + stage * (bStageBytes >> 4);
                    const bool cross = Tf32 && it < kbCount;
                    #pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                    {
                        const uint64_t da = descHiA | static_cast<uint64_t>(aLo + j * advA);
                        const uint64_t db = descHiB | static_cast<uint64_t>(bLo + j * advB);
                        if (cross) umma<false>(tmemD, da, db, idesc16, (it | j) != 0 ? 1u : 0u);
                        else       umma<Tf32>(tmemD, da, db, idesc, (it | j) != 0 ? 1u : 0u);
                    }
                    ummaCommit(&s.empty[stage]);           // the stage is free once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ummaCommit(&s.tmemFull[acc]);       // accumulator complete
                acc ^= 1u;
                if (acc == 0) accPhase ^= 1u;
            }
        }
    }
    else
    {
        // Epilogue warps 2..5 own TMEM lanes 32*(warp % 4) .. +31, i.e. rows of the tile.
        const uint32_t quarter = warp & 3u;
        uint32_t acc = 0, accPhase = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < totalTiles && ok; t += gridDim.x)
        {
            uint32_t tm, tn;
            tileCoordinates(t, p.tilesM, p.tilesN, p.tileGroup, tm, tn);
            for (uint32_t c = 0; c < p.chunks && ok; ++c)
            {
            if (!mbarWait(&s.tmemFull[acc], accPhase, abortFlag)) { ok = false; break; }
            fenceAfterSync();
            const uint32_t row = tm * kBlockM + quarter * 32 + lane;
            const uint32_t taddr = tmemBase + acc * kBlockN + ((quarter * 32u) << 16);
            drainAccumulator(p, taddr, row, tn * p.blockN, c);
            fenceBeforeSync();
            mbarArrive(&s.tmemEmpty[acc]);
            acc ^= 1u;
            if (acc == 0) accPhase ^= 1u;
            }
        }
    }

    if (threadIdx.x == 0) lingerAfterAbort(abortFlag);
    fenceBeforeSync();
    __syncthreads();
    if (warp == 1)
    {
        fenceAfterSync();
        tmemDealloc(tmemBase, kTmemColumns);
    }
    if (threadIdx.x == 0 && s.abortFlag) atomicExch(p.errorWord, 1u);
}

// ==================================================================================================================
// CTA-pair variant (cta_group::2). Two CTAs of a cluster own one 256 x 256 tile: CTA r holds rows r*128.. of A and of
// the accumulator, and columns r*128.. of B; the leader CTA (rank 0) issues M=256 MMAs that read both CTAs' shared
// memory. Each CTA therefore loads 32 KiB per stage instead of 48 KiB, which buys a 6-stage ring: the single-CTA
// kernel stalls on TMA latency with its 4 stages (tensor pipe 56 % busy at 4096^3). No TMA multicast is used: every
// CTA loads its own operand slices and signals the leader's `full` barrier (cp.async.bulk.tensor ... .cta_group::2).
// ==================================================================================================================
// Work distribution of the pair kernel. A persistent grid loses the idle part of its last wave of tiles (256 tiles on
// 74 clusters: 3.46 waves cost 4). The remainder tiles [0, splitTiles) are therefore cut along K into `splitUnits`
// k-blocks that are dealt out evenly: cluster i takes units [i*U/C, (i+1)*U/C), a range shorter than one tile, i.e.
// the tail of one tile followed by the head of the next. These pieces come FIRST in every cluster's sequence, the whole
// tiles [splitTiles, tiles) follow round-robin. The cluster that owns the head of a tile (k-block 0) finishes it: the
// others publish their f32 partial accumulators in a workspace slot of their own and bump a counter; the finisher -
// which reaches that piece last in its own range, when the others are normally long done - waits for the counter,
// adds the partials in cluster order (deterministic) and stores C. Nobody ever waits for the finisher, so the wait
// cannot cycle; it is bounded in time like every other wait of the kernel.
enum : uint32_t { kWorkWhole = 0, kWorkPartial = 1, kWorkFinish = 2 };
struct WorkItem
{
    uint32_t tile, kbBegin, kbCount, kind;
    uint32_t partials;          // kWorkFinish: accumulators of the following `partials` clusters belong to this tile
};
// Which tiles a cluster computes. Static deal (tileCounters == null, and always for problems whose remainder wave is cut
// along K): cluster c takes tiles c, c + clusters, ... Dynamic deal: one thread of the cluster - the leader CTA's TMA producer,
// the first to need the answer - draws the next tile from a device-wide counter and publishes it, tagged with the launch and
// the iteration, in the cluster's ring in global memory; every other role of both CTAs reads it there (a bounded spin; one
// 8-byte load per tile and role). A cluster that starts late - because a collective's kernel held its SMs when the matmul
// was launched - then simply draws fewer tiles, instead of finishing a fixed share late and the whole product with it. The
// producer draws one tile ahead, so the counter's latency stays off its path.
constexpr uint32_t kNoTile = 0xFFFFFu;
enum : uint32_t { kRoleFetcher = 0, kRoleThread = 1, kRoleWarp = 2 };
struct WorkIterator
{
    uint32_t cluster, clusters, kBlocks, tiles, unit, unitEnd, units, next;
    // dynamic deal
    uint32_t* counter = nullptr;
    uint64_t* ring = nullptr;
    uint64_t  tagBase = 0;
    uint32_t  role = kRoleThread, iteration = 0, drawn = kNoTile;
    volatile uint32_t* abortFlag = nullptr;

    __device__ WorkIterator(const KernelParams& p, uint32_t clusterId, uint32_t clusterCount, uint32_t roleOfCaller = kRoleThread,
                            volatile uint32_t* abort = nullptr)
        : cluster(clusterId), clusters(clusterCount), kBlocks(p.kBlocks), tiles(p.tilesM * p.tilesN),
          unit(static_cast<uint32_t>(static_cast<uint64_t>(clusterId) * p.splitUnits / clusterCount)),
          unitEnd(static_cast<uint32_t>(static_cast<uint64_t>(clusterId + 1) * p.splitUnits / clusterCount)),
          units(p.splitUnits), next(p.splitTiles + clusterId)
    {
        if (p.tileCounters)
        {
            counter = p.tileCounters + (p.tileEpoch & 7u) * 16u;
            ring = p.tileRing + static_cast<size_t>(clusterId) * kernels::kGemmRingSlots;
            tagBase = static_cast<uint64_t>(p.tileEpoch) << 40;
            role = roleOfCaller;
            abortFlag = abort;
            if (role == kRoleFetcher)
            {
                if (clusterId == 0) p.tileCounters[((p.tileEpoch + 4u) & 7u) * 16u] = 0;     // ready for the launch four launches on
                drawn = atomicAdd(counter, 1u);
            }
        }
    }
    __device__ uint32_t await(uint64_t tag)
    {
        const uint64_t* slot = ring + (iteration % kernels::kGemmRingSlots);
        const uint64_t start = globalTimerNs();
        uint32_t spins = 0;
        for (;;)
        {
            uint64_t v;
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot) : "memory");
            if ((v >> 20) == (tag >> 20)) return static_cast<uint32_t>(v & 0xFFFFFu);
            if ((++spins & 63u) == 0)
            {
                if (*abortFlag) return kNoTile;
                if (globalTimerNs() - start > kWaitLimitNs) { *abortFlag = 1; return kNoTile; }
            }
        }
    }
    __device__ bool get(WorkItem& w)
    {
        if (counter)
        {
            const uint64_t tag = tagBase | (static_cast<uint64_t>(iteration) << 20);
            uint32_t tile;
            if (role == kRoleFetcher)
            {
                tile = drawn < tiles ? drawn : kNoTile;
                asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(ring + (iteration % kernels::kGemmRingSlots)), "l"(tag | tile) : "memory");
                if (tile != kNoTile) drawn = atomicAdd(counter, 1u);        // the next one, needed a whole tile from now
            }
            else if (role == kRoleThread) tile = await(tag);
            else
            {
                // the lanes that are here together (all 32 unless a wait gave up in some of them): the first one reads
                const uint32_t together = __activemask(), first = static_cast<uint32_t>(__ffs(static_cast<int>(together))) - 1u;
                tile = (threadIdx.x & 31u) == first ? await(tag) : 0u;
                tile = __shfl_sync(together, tile, static_cast<int>(first));
            }
            ++iteration;
            if (tile == kNoTile) return false;
            w.tile = tile; w.kbBegin = 0; w.kbCount = kBlocks; w.kind = kWorkWhole; w.partials = 0;
            return true;
        }
        if (unit < unitEnd)
        {
            w.tile = unit / kBlocks;
            w.kbBegin = unit - w.tile * kBlocks;
            w.kbCount = min(kBlocks - w.kbBegin, unitEnd - unit);
            w.partials = 0;
            if (w.kbCount == kBlocks) w.kind = kWorkWhole;
            else if (w.kbBegin != 0) w.kind = kWorkPartial;
            else
            {
                // the cluster whose range holds the tile's last unit u: the largest j with floor(j*U/C) <= u
                const uint64_t u = static_cast<uint64_t>(w.tile + 1) * kBlocks - 1;
                const uint32_t last = static_cast<uint32_t>(((u + 1) * clusters - 1) / units);
                w.kind = kWorkFinish;
                w.partials = last - cluster;
            }
            unit += w.kbCount;
            return true;
        }
        if (next < tiles)
        {
            w.tile = next; w.kbBegin = 0; w.kbCount = kBlocks; w.kind = kWorkWhole; w.partials = 0;
            next += clusters;
            return true;
        }
        return false;
    }
};

__device__ __forceinline__ void epilogueBarrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // warps 2..5 only

// kWorkPartial: the accumulator row of this thread goes to the cluster's workspace slot as f32.
__device__ __forceinline__ void publishPartial(const KernelParams& p, uint32_t taddr, float* slotRow)
{
    #pragma unroll 1
    for (uint32_t c0 = 0; c0 < p.blockN; c0 += 64)
    {
        uint32_t r0[32], r1[32];
        tmemLoad32(taddr + c0, r0);
        tmemLoad32(taddr + c0 + 32, r1);
        tmemLoadWait();
        float4* out = reinterpret_cast<float4*>(slotRow + c0);
        #pragma unroll
        for (int v = 0; v < 8; ++v)
            out[v] = make_float4(__uint_as_float(r0[4 * v]), __uint_as_float(r0[4 * v + 1]), __uint_as_float(r0[4 * v + 2]), __uint_as_float(r0[4 * v + 3]));
        #pragma unroll
        for (int v = 0; v < 8; ++v)
            out[8 + v] = make_float4(__uint_as_float(r1[4 * v]), __uint_as_float(r1[4 * v + 1]), __uint_as_float(r1[4 * v + 2]), __uint_as_float(r1[4 * v + 3]));
    }
}

// kWorkFinish: own accumulator plus the partials of the following clusters (read through L2), then the usual store.
__device__ __forceinline__ void finishTile(const KernelParams& p, uint32_t taddr, uint32_t row, uint32_t colBase, const float* firstSlotRow,
                                           size_t slotStride, uint32_t partials)
{
    const float4 unusedOld[8] = {};
    #pragma unroll 1
    for (uint32_t c0 = 0; c0 < p.blockN; c0 += 32)
    {
        uint32_t r[32];
        tmemLoad32(taddr + c0, r);
        tmemLoadWait();
        for (uint32_t j = 0; j < partials; ++j)
        {
            const float4* in = reinterpret_cast<const float4*>(firstSlotRow + j * slotStride + c0);
            #pragma unroll
            for (int v = 0; v < 8; ++v)
            {
                const float4 x = __ldcg(in + v);
                r[4 * v]     = __float_as_uint(__uint_as_float(r[4 * v]) + x.x);
                r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + x.y);
                r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + x.z);
                r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + x.w);
            }
        }
        storeAccumulatorRow(p, r, unusedOld, row, colBase + c0, 0);
    }
}

// One stage of the pair kernel holds TWO 128-byte swizzle atoms along K per operand (128 16-bit or 64 TF32 elements of
// K): fetched as ONE 3-D TMA box, every operand row (or K line of an MN-major operand) is then a 256-byte contiguous run
// in global memory. Measured: MN-major operands loaded as two 64 x 64 boxes ran A.B at 1006 and A^T.B at 887 TFLOP/s
// (4096^3 bf16); as one 3-D box each, at 1325 and 1411 - above the all-K-major form with its 128-byte runs (1182).
constexpr int kPairStages = 3;
constexpr int kPairStageBytesA = 128 * 256;
constexpr int kPairStageBytesB = 128 * 256;
constexpr int kWarpStagingBytes = 32 * 128;

struct PairStorage
{
    alignas(1024) uint8_t a[kPairStages][kPairStageBytesA];
    alignas(1024) uint8_t b[kPairStages][kPairStageBytesB];
    uint64_t full[kPairStages];        // used in the leader CTA: both CTAs' loads land here
    uint64_t empty[kPairStages];       // one per CTA, released by the leader's multicast commit
    uint64_t tmemFull[2];              // one per CTA, multicast commit
    uint64_t tmemEmpty[2];             // used in the leader CTA: 256 epilogue threads of the pair arrive
    uint32_t tmemBase;
    uint32_t abortFlag;
    alignas(1024) uint8_t staging[4][2 * kWarpStagingBytes];   // epilogue: per warp two buffers of 32 rows x 128 bytes, swizzled, for TMA stores
};

__device__ __forceinline__ uint32_t clusterRank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapToCta(uint32_t sharedAddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(sharedAddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void clusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbarExpectTxCluster(uint32_t clusterAddr, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(clusterAddr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
__device__ __forceinline__ void tmaLoad2dPair(void* dst, const CUtensorMap* map, uint32_t leaderBar, int32_t c0, int32_t c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smemAddr(dst)), "l"(map), "r"(leaderBar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmaLoad3dPair(void* dst, const CUtensorMap* map, uint32_t leaderBar, int32_t c0, int32_t c1, int32_t c2)
{
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smemAddr(dst)), "l"(map), "r"(leaderBar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
template <bool Tf32>
__device__ __forceinline__ void ummaPair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    if (Tf32)
        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n}"
                     ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                     ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ummaCommitPair(uint64_t* bar)
{
    // arrives on the barrier at this offset in BOTH CTAs of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smemAddr(bar)), "h"(static_cast<uint16_t>(3)) : "memory");
}

// ---- epilogue through shared memory and TMA ---------------------------------------------------------------------------
// The direct epilogue has every thread store its own accumulator row: each warp-wide 16-byte store touches 32
// different 128-byte lines, and for split-f32 problems every partial sum also READS C that way. Those accesses share
// the L1 / shared-memory pipe with the TMA loads and the tensor core's operand reads (measured: l1tex throughput 77 % in
// the f32 kernel). Here a slice of 128 rows x 128 bytes is written to shared memory in the 128-byte swizzle (conflict
// free: 4 wavefronts per warp store), and one thread hands it to the TMA unit: a tile store for the first partial
// sum, an f32 reduce-add (performed in L2, IEEE round-to-nearest) for the later ones, so C is never loaded by the SM.
// The TMA unit also clips rows >= M and columns >= N. Partial sums of one tile are ordered by waiting for the earlier
// bulk groups to complete before the next partial sum's first reduce-add is issued.
__device__ __forceinline__ void tmaStoreTile(const CUtensorMap* map, const void* src, int32_t x, int32_t y, bool reduceAdd)
{
    if (reduceAdd)
        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                     ::"l"(map), "r"(smemAddr(src)), "r"(x), "r"(y) : "memory");
    else
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                     ::"l"(map), "r"(smemAddr(src)), "r"(x), "r"(y) : "memory");
}

// One 32-row x 128-byte slice of C leaves through this warp's own staging buffer: no barrier wider than the warp.
__device__ __forceinline__ void emitSlice(const CUtensorMap* mapC, uint8_t* warpStaging, uint32_t& sliceCounter, const uint4 (&chunks)[8],
                                          uint32_t lane, int32_t x, int32_t y, bool reduceAdd)
{
    uint8_t* buffer = warpStaging + (sliceCounter & 1u) * kWarpStagingBytes;
    // the TMA operation that used this buffer two slices ago must have read it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
    uint8_t* rowPtr = buffer + lane * 128u;
    const uint32_t swizzle = lane & 7u;
    #pragma unroll
    for (uint32_t v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(rowPtr + ((v ^ swizzle) << 4)) = chunks[v];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // generic-proxy writes -> visible to the TMA unit
    __syncwarp();
    if (lane == 0)
    {
        tmaStoreTile(mapC, buffer, x, y, reduceAdd);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    ++sliceCounter;
}

__device__ __forceinline__ void packF32(const uint32_t (&r)[32], uint4 (&chunks)[8], float scaleA, float scaleB)
{
    // the two factors are applied one after the other: their product may leave the float range when the result does not
    #pragma unroll
    for (int v = 0; v < 8; ++v)
        chunks[v] = make_uint4(__float_as_uint(__uint_as_float(r[4 * v]) * scaleA * scaleB), __float_as_uint(__uint_as_float(r[4 * v + 1]) * scaleA * scaleB),
                               __float_as_uint(__uint_as_float(r[4 * v + 2]) * scaleA * scaleB), __float_as_uint(__uint_as_float(r[4 * v + 3]) * scaleA * scaleB));
}

// `taddr` addresses this warp's 32 TMEM lanes; (x0, y0) is the position in C of their first element.
__device__ __forceinline__ void drainAccumulatorTma(const KernelParams& p, const CUtensorMap* mapC, uint8_t* warpStaging, uint32_t& sliceCounter,
                                                    uint32_t taddr, uint32_t lane, int32_t x0, int32_t y0, uint32_t c)
{
    const bool reduceAdd = c > 0;
    if (lane == 0 && reduceAdd) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // earlier partial sums of these rows have landed
    if (p.outDtype == F32)
    {
        // 32 columns per slice; the TMEM load of the next slice is in flight while this one is staged and handed over
        uint32_t rA[32], rB[32];
        uint4 chunks[8];
        const float scaleA = p.halfTerms ? halfTermInverseScale(*p.scaleA) : 1.0f;      // multiplying by 1 is exact
        const float scaleB = p.halfTerms ? halfTermInverseScale(*p.scaleB) : 1.0f;
        tmemLoad32(taddr, rA);
        #pragma unroll 1
        for (uint32_t c0 = 0; c0 < p.blockN; c0 += 64)
        {
            tmemLoadWait();
            tmemLoad32(taddr + c0 + 32, rB);
            packF32(rA, chunks, scaleA, scaleB);
            emitSlice(mapC, warpStaging, sliceCounter, chunks, lane, x0 + static_cast<int32_t>(c0), y0, reduceAdd);
            tmemLoadWait();
            if (c0 + 64 < p.blockN) tmemLoad32(taddr + c0 + 64, rA);
            packF32(rB, chunks, scaleA, scaleB);
            emitSlice(mapC, warpStaging, sliceCounter, chunks, lane, x0 + static_cast<int32_t>(c0 + 32), y0, reduceAdd);
        }
        return;
    }
    #pragma unroll 1
    for (uint32_t c0 = 0; c0 < p.blockN; c0 += 64)                    // 64 columns of 16-bit output per slice
    {
        uint32_t r0[32], r1[32];
        tmemLoad32(taddr + c0, r0);
        tmemLoad32(taddr + c0 + 32, r1);
        tmemLoadWait();
        uint32_t packed[32];
        #pragma unroll
        for (int v = 0; v < 16; ++v)
        {
            const float a0 = __uint_as_float(r0[2 * v]), a1 = __uint_as_float(r0[2 * v + 1]);
            const float b0 = __uint_as_float(r1[2 * v]), b1 = __uint_as_float(r1[2 * v + 1]);
            if (p.outDtype == BF16)
            {
                packed[v] = static_cast<uint32_t>(dev::f32ToBf16(a0)) | (static_cast<uint32_t>(dev::f32ToBf16(a1)) << 16);
                packed[16 + v] = static_cast<uint32_t>(dev::f32ToBf16(b0)) | (static_cast<uint32_t>(dev::f32ToBf16(b1)) << 16);
            }
            else
            {
                packed[v] = static_cast<uint32_t>(dev::f32ToF16(a0)) | (static_cast<uint32_t>(dev::f32ToF16(a1)) << 16);
                packed[16 + v] = static_cast<uint32_t>(dev::f32ToF16(b0)) | (static_cast<uint32_t>(dev::f32ToF16(b1)) << 16);
            }
        }
        uint4 chunks[8];
        #pragma unroll
        for (int v = 0; v < 8; ++v) chunks[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
        emitSlice(mapC, warpStaging, sliceCounter, chunks, lane, x0 + static_cast<int32_t>(c0), y0, false);
    }
}

// tanh of the folded epilogue: the same routine the generated elementwise kernels use in their default math mode, so a
// product whose bias and tanh are folded into the matmul gives the bits the separate kernels would give.
// |x| < 0.6: x + x^3 * p(x^2), a degree-4 fit of (tanh(x) - x) / x^3 (max relative error 9e-8); otherwise
// 1 - 2 / (exp(2|x|) + 1) with the sign of x.
__device__ __forceinline__ float epilogueTanh(float x)
{
    const float t = fabsf(x), u = x * x;
    float q = -0.006276384927332401f;
    q = fmaf(q, u, 0.021116212010383606f);
    q = fmaf(q, u, -0.053875137120485306f);
    q = fmaf(q, u, 0.13332924246788025f);
    q = fmaf(q, u, -0.3333333134651184f);
    const float small = fmaf(x * u, q, x);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t * 2.885390081777927f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
    const float large = copysignf(fmaf(-2.0f, r, 1.0f), x);
    return t < 0.6f ? small : large;
}

// Mode 0: 16-bit operands, one pass. Mode 1: f32 as a TF32 main pass plus two bf16 cross-term passes. Mode 2: f32 as three
// fp16 passes over two-term operands - every pass is a 16-bit pass, so nothing in the issue loops depends on the pass.
// Modes 3 and 4: mode 2 with elementwise consumers folded into the epilogue - the bias add (3), and its tanh as well (4);
// instantiations of their own, so that the plain product and the add-only form keep their register allocation.
template <int Mode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Mode >= 2 ? kThreadsHalfTerms : kThreads, 1)
gemmPairKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapA16,
               const __grid_constant__ CUtensorMap mapB16, const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapC1,
               const __grid_constant__ CUtensorMap mapC2, const __grid_constant__ KernelParams p)
{
    constexpr bool Tf32 = Mode != 0;
    constexpr bool HalfTerms = Mode >= 2;
    constexpr bool Fold = Mode >= 3;             // consumers folded into the epilogue: the bias add (3), and its tanh (4)
    constexpr bool FoldTanh = Mode == 4;
    extern __shared__ uint8_t rawSmem[];
    PairStorage& s = *reinterpret_cast<PairStorage*>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = clusterRank();
    const bool leader = rank == 0;
    volatile uint32_t* abortFlag = &s.abortFlag;

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < kPairStages; ++i) { mbarInit(&s.full[i], 2); mbarInit(&s.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbarInit(&s.tmemFull[i], 1); mbarInit(&s.tmemEmpty[i], HalfTerms ? 512 : 256); }   // epilogue threads of the pair
        s.abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&s.tmemBase)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    fenceBeforeSync();
    __syncthreads();
    clusterSync();                      // barriers of both CTAs are initialised before anyone signals across
    fenceAfterSync();
    const uint32_t tmemBase = s.tmemBase;
    const uint32_t clusterId = blockIdx.x >> 1, clusters = gridDim.x >> 1;

    if (warp == 0)
    {
        if (lane == 0)
        {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint32_t stageBytes = p.pairABytes + p.pairBBytes;
            const uint32_t leaderFull0 = mapToCta(smemAddr(&s.full[0]), 0);
            WorkIterator work(p, clusterId, clusters, leader ? kRoleFetcher : kRoleThread, abortFlag);
            WorkItem w;
            while (ok && work.get(w))
            {
                uint32_t tm, tn;
                tileCoordinates(w.tile, p.tilesM, p.tilesN, p.tileGroup, tm, tn);
                const int32_t m0 = static_cast<int32_t>(tm * 256 + rank * 128), n0 = static_cast<int32_t>(tn * p.blockN + rank * (p.blockN >> 1));
                for (uint32_t c = 0; c < p.chunks && ok; ++c)
                {
                    const uint32_t kbBegin = w.kbBegin + c * p.chunkBlocks, kbCount = min(w.kbBegin + w.kbCount - kbBegin, p.chunkBlocks);
                    for (uint32_t passIndex = 0; passIndex < p.kPhases && ok; ++passIndex)
                    {
                    // hybrid scheme: two bf16 cross-term passes (stages of 128) before the TF32 main pass (stages of 64);
                    // half-term scheme: three fp16 passes, all with stages of 128 (h1.h0', h0.h1', h0.h0')
                    const bool cross = Tf32 && (passIndex < 2 || HalfTerms);
                    const bool halved = cross && !HalfTerms;
                    const uint32_t first = halved ? kbBegin >> 1 : kbBegin, count = halved ? kbCount >> 1 : kbCount;
                    const uint32_t atomK = cross ? 64u : p.atomK;
                    const CUtensorMap* ma = cross ? &mapA16 : &mapA;
                    const CUtensorMap* mb = cross ? &mapB16 : &mapB;
                    // the second term (or `lo` part) of a split-f32 operand lies one plane further: along K when the operand
                    // is K-major, along its M / N dimension when it is MN-major
                    const uint32_t offA = (cross && passIndex == 0) ? p.aPlane : 0u, offB = (cross && passIndex == 1) ? p.bPlane : 0u;
                    const uint32_t offKA = p.aMnMajor ? 0u : offA, offKB = p.bMnMajor ? 0u : offB;
                    const int32_t m0p = m0 + static_cast<int32_t>(p.aMnMajor ? offA : 0u), n0p = n0 + static_cast<int32_t>(p.bMnMajor ? offB : 0u);
                    for (uint32_t kb = first; kb < first + count; ++kb)
                    {
                        if (!mbarWait(&s.empty[stage], phase ^ 1u, abortFlag)) { ok = false; break; }
                        const uint32_t leaderFull = leaderFull0 + stage * 8;
                        mbarExpectTxCluster(leaderFull, stageBytes);
                        const uint32_t kA = kb * 2 * atomK + offKA, kB = kb * 2 * atomK + offKB;
                        if (p.aMnMajor)
                        {
                            if (p.aLoad3d) tmaLoad3dPair(&s.a[stage][0], ma, leaderFull, 0, static_cast<int32_t>(kA), m0p >> 6);
                            else for (uint32_t at = 0; at < 2; ++at) for (uint32_t h = 0; h < 2; ++h)
                                tmaLoad2dPair(&s.a[stage][at * 16384 + h * 8192], ma, leaderFull, m0 + static_cast<int32_t>(at * 64), static_cast<int32_t>(kA + h * 64));
                        }
                        else
                        {
                            if (p.aLoad3d) tmaLoad3dPair(&s.a[stage][0], ma, leaderFull, 0, m0, static_cast<int32_t>(kA / atomK));
                            else for (uint32_t h = 0; h < 2; ++h)
                                tmaLoad2dPair(&s.a[stage][h * (p.pairABytes >> 1)], ma, leaderFull, static_cast<int32_t>(kA + h * atomK), m0);
                        }
                        if (p.bMnMajor)
                        {
                            if (p.bLoad3d) tmaLoad3dPair(&s.b[stage][0], mb, leaderFull, 0, static_cast<int32_t>(kB), n0p >> 6);
                            else for (uint32_t at = 0; at < (p.blockN >> 7); ++at) for (uint32_t h = 0; h < 2; ++h)
                                tmaLoad2dPair(&s.b[stage][at * 16384 + h * 8192], mb, leaderFull, n0 + static_cast<int32_t>(at * 64), static_cast<int32_t>(kB + h * 64));
                        }
                        else
                        {
                            if (p.bLoad3d) tmaLoad3dPair(&s.b[stage][0], mb, leaderFull, 0, n0, static_cast<int32_t>(kB / atomK));
                            else for (uint32_t h = 0; h < 2; ++h)
                                tmaLoad2dPair(&s.b[stage][h * (p.pairBBytes >> 1)], mb, leaderFull, static_cast<int32_t>(kB + h * atomK), n0);
                        }
                        if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                    }
                    }
                }
            }
        }
    }
    else if (warp == 1)
    {
        if (lane == 0 && leader)
        {
            // Descriptor halves that never change: the high word (stride offsets, version, swizzle) and the low word of
            // stage 0; per stage and per MMA only a 32-bit add remains.
            const uint64_t descHiA = smemDescriptor(0, p.pairALbo, 1024), descHiB = smemDescriptor(0, p.pairBLbo, 1024);
            const uint32_t descLoA = (smemAddr(&s.a[0][0]) & 0x3FFFFu) >> 4, descLoB = (smemAddr(&s.b[0][0]) & 0x3FFFFu) >> 4;
            const uint32_t aStageBytes = sizeof(s.a[0]), bStageBytes = sizeof(s.b[0]);
            const uint32_t idesc = p.idesc, idesc16 = p.idesc16;
            uint32_t aOff[8], bOff[8];
            #pragma unroll
            for (int j = 0; j < 8; ++j) { aOff[j] = p.pairAOff[j]; bOff[j] = p.pairBOff[j]; }
            uint32_t stage = 0, phase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            WorkIterator work(p, clusterId, clusters, kRoleThread, abortFlag);
            WorkItem w;
            while (ok && work.get(w))
            for (uint32_t c = 0; c < p.chunks && ok; ++c)
            {
                if (!mbarWait(&s.tmemEmpty[acc], accPhase ^ 1u, abortFlag)) { ok = false; break; }
                fenceAfterSync();
                const uint32_t tmemD = tmemBase + acc * kBlockN;
                const uint32_t kbCount = min(w.kbCount - c * p.chunkBlocks, p.chunkBlocks);
                // f32 problems: kbCount bf16 stages (two cross-term passes of kbCount / 2 stages of 128), then kbCount
                // TF32 stages of 64
                const uint32_t stagesInChunk = Tf32 ? (HalfTerms ? 3 * kbCount : 2 * kbCount) : kbCount;
                for (uint32_t it = 0; it < stagesInChunk; ++it)
                {
                    if (!mbarWait(&s.full[stage], phase, abortFlag)) { ok = false; break; }
                    fenceAfterSync();
                    const uint32_t aLo = descLoA + stage * (aStageBytes >> 4), bLo = descLoB + stage * (bStageBytes >> 4);
                    const bool cross = Tf32 && (HalfTerms || it < kbCount);
                    #pragma unroll
                    for (uint32_t j = 0; j < 8; ++j)
                    {
                        const uint64_t da = descHiA | static_cast<uint64_t>(aLo + aOff[j]);
                        const uint64_t db = descHiB | static_cast<uint64_t>(bLo + bOff[j]);
                        if (HalfTerms || cross) ummaPair<false>(tmemD, da, db, idesc16, (it | j) != 0 ? 1u : 0u);
                        else                    ummaPair<Tf32>(tmemD, da, db, idesc, (it | j) != 0 ? 1u : 0u);
                    }
                    ummaCommitPair(&s.empty[stage]);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) ummaCommitPair(&s.tmemFull[acc]);
                acc ^= 1u;
                if (acc == 0) accPhase ^= 1u;
            }
        }
    }
    else
    {
        if constexpr (HalfTerms)
        {
            // f32 as three fp16 passes: K is cut into chunks whose partial sums must be added in IEEE f32 (the tensor core's
            // own accumulation truncates). The running sum of the tile lives in REGISTERS: eight epilogue warps - two per
            // TMEM lane quarter, each owning half of the tile's columns - read every finished chunk from TMEM and add it to
            // 32 rows x (blockN / 2) columns of sums, one row per thread. Nothing leaves the SM until the tile is complete;
            // then the sums are scaled back and stored once through shared memory and TMA (or directly when C's rows are
            // not 16-byte aligned). Per chunk the epilogue costs four TMEM loads and 128 additions per thread, so it never
            // holds an accumulator long enough to stall the MMA issue.
            const uint32_t ewarp = warp - 2u, quarter = warp & 3u, half = ewarp >> 2;
            const uint32_t halfCols = p.blockN >> 1;                         // 128, or 64 for narrow tiles
            uint8_t* staging = &s.staging[0][0] + ewarp * kWarpStagingBytes; // one 32 x 128-byte buffer per warp
            float sum[128];
            uint32_t acc = 0, accPhase = 0;
            bool ok = true;
            WorkIterator work(p, clusterId, clusters, kRoleWarp, abortFlag);
            WorkItem w;
            while (ok && work.get(w))
            {
                uint32_t tm, tn;
                tileCoordinates(w.tile, p.tilesM, p.tilesN, p.tileGroup, tm, tn);
                const uint32_t leaderEmpty = mapToCta(smemAddr(&s.tmemEmpty[0]), 0);
                for (uint32_t c = 0; c < p.chunks && ok; ++c)
                {
                    if (!mbarWait(&s.tmemFull[acc], accPhase, abortFlag)) { ok = false; break; }
                    fenceAfterSync();
                    const uint32_t taddr = tmemBase + acc * kBlockN + ((quarter * 32u) << 16) + half * halfCols;
                    #pragma unroll
                    for (uint32_t strip = 0; strip < 8; ++strip)         // 16 columns per TMEM load: the sums leave few registers to spare
                    {
                        if (strip * 16 < halfCols)
                        {
                            uint32_t r[16];
                            tmemLoad16(taddr + strip * 16, r);
                            tmemLoadWait();
                            #pragma unroll
                            for (int i = 0; i < 16; ++i) sum[strip * 16 + i] = (c == 0) ? __uint_as_float(r[i]) : sum[strip * 16 + i] + __uint_as_float(r[i]);
                        }
                    }
                    fenceBeforeSync();
                    mbarArriveCluster(leaderEmpty + acc * 8);
                    acc ^= 1u;
                    if (acc == 0) accPhase ^= 1u;
                }
                if (!ok) break;
                // the tile is complete: undo the operands' scaling (two exact factors, one after the other) and store.
                // Elementwise consumers folded into this epilogue (p.outputs) take the values from the same registers:
                // C + bias and tanh(C + bias) leave through their own tensor maps, and C itself only if somebody reads it.
                const float scaleA = halfTermInverseScale(*p.scaleA), scaleB = halfTermInverseScale(*p.scaleB);
                const uint32_t col0 = tn * p.blockN + half * halfCols;
                const uint32_t row0 = tm * 256 + rank * 128 + quarter * 32;
                const uint32_t outputs = Fold ? p.outputs : 1u;
                uint32_t maxBits = 0;
                #pragma unroll
                for (uint32_t strip = 0; strip < 4; ++strip)
                {
                    if (strip * 32 >= halfCols) continue;
                    #pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) sum[strip * 32 + i] = sum[strip * 32 + i] * scaleA * scaleB;
                    if (p.tmaEpilogue)
                    {
                        auto stageAndStore = [&](const CUtensorMap* map)
                        {
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // the buffer's previous slice has been read
                            __syncwarp();
                            uint8_t* rowPtr = staging + lane * 128u;
                            const uint32_t swizzle = lane & 7u;
                            #pragma unroll
                            for (uint32_t v = 0; v < 8; ++v)
                                *reinterpret_cast<uint4*>(rowPtr + ((v ^ swizzle) << 4)) =
                                    make_uint4(__float_as_uint(sum[strip * 32 + 4 * v]), __float_as_uint(sum[strip * 32 + 4 * v + 1]),
                                               __float_as_uint(sum[strip * 32 + 4 * v + 2]), __float_as_uint(sum[strip * 32 + 4 * v + 3]));
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if (lane == 0)
                            {
                                tmaStoreTile(map, staging, static_cast<int32_t>(col0 + strip * 32), static_cast<int32_t>(row0), false);
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            }
                        };
                        if (outputs & 1u) stageAndStore(&mapC);
                        if constexpr (Fold) if (outputs & 6u)
                        {
                            const uint32_t colS = col0 + strip * 32;
                            #pragma unroll
                            for (uint32_t v = 0; v < 8; ++v)
                            {
                                // every lane reads the same four bias values: one broadcast load; n is a multiple of 4
                                const float4 bv = colS + 4 * v < p.n ? __ldg(reinterpret_cast<const float4*>(p.bias + colS + 4 * v)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                                sum[strip * 32 + 4 * v] += bv.x; sum[strip * 32 + 4 * v + 1] += bv.y;
                                sum[strip * 32 + 4 * v + 2] += bv.z; sum[strip * 32 + 4 * v + 3] += bv.w;
                            }
                            if (outputs & 2u) stageAndStore(&mapC1);
                            if constexpr (FoldTanh) if (outputs & 4u)
                            {
                                #pragma unroll
                                for (uint32_t i = 0; i < 32; ++i) sum[strip * 32 + i] = epilogueTanh(sum[strip * 32 + i]);
                                stageAndStore(&mapC2);
                            }
                            if (p.maxSlot && row0 + lane < p.m)
                            {
                                #pragma unroll
                                for (uint32_t i = 0; i < 32; ++i)
                                    if (colS + (i & ~3u) < p.n) maxBits = max(maxBits, __float_as_uint(sum[strip * 32 + i]) & 0x7FFFFFFFu);
                            }
                        }
                    }
                    else
                    {
                        const uint32_t row = row0 + lane;
                        if (row < p.m)
                        {
                            float* out = static_cast<float*>(p.c) + static_cast<size_t>(row) * p.n;
                            #pragma unroll
                            for (uint32_t i = 0; i < 32; ++i)
                            {
                                const uint32_t col = col0 + strip * 32 + i;
                                if (col < p.n) out[col] = sum[strip * 32 + i];
                            }
                        }
                    }
                }
                if constexpr (Fold) if (p.maxSlot)
                {
                    // the bit patterns of non-negative floats order like the floats, and a NaN's lies above every number's
                    maxBits = __reduce_max_sync(0xFFFFFFFFu, maxBits);
                    if (lane == 0 && maxBits != 0) atomicMax(p.maxSlot, maxBits);
                }
            }
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // staging buffers are read, C is written
        }
        else
        {
        const uint32_t quarter = warp & 3u;
        const bool captain = threadIdx.x == 64;                          // first thread of the epilogue warps
        const uint32_t rowInCta = quarter * 32 + lane;
        const size_t slotStride = size_t(2) * 128 * 256;                 // floats per cluster slot of the workspace
        uint32_t acc = 0, accPhase = 0, sliceCounter = 0;
        bool ok = true;
        WorkIterator work(p, clusterId, clusters, kRoleWarp, abortFlag);
        WorkItem w;
        while (ok && work.get(w))
        {
            uint32_t tm, tn;
            tileCoordinates(w.tile, p.tilesM, p.tilesN, p.tileGroup, tm, tn);
            const uint32_t row = tm * 256 + rank * 128 + rowInCta;
            const uint32_t leaderEmpty = mapToCta(smemAddr(&s.tmemEmpty[0]), 0);
            if (w.kind == kWorkWhole)
            {
                for (uint32_t c = 0; c < p.chunks && ok; ++c)
                {
                    if (!mbarWait(&s.tmemFull[acc], accPhase, abortFlag)) { ok = false; break; }
                    fenceAfterSync();
                    const uint32_t taddr = tmemBase + acc * kBlockN + ((quarter * 32u) << 16);
                    if (p.tmaEpilogue)
                        drainAccumulatorTma(p, &mapC, s.staging[quarter], sliceCounter, taddr, lane, static_cast<int32_t>(tn * p.blockN),
                                            static_cast<int32_t>(tm * 256 + rank * 128 + quarter * 32), c);
                    else
                        drainAccumulator(p, taddr, row, tn * p.blockN, c);
                    fenceBeforeSync();
                    mbarArriveCluster(leaderEmpty + acc * 8);
                    acc ^= 1u;
                    if (acc == 0) accPhase ^= 1u;
                }
                continue;
            }
            if (!mbarWait(&s.tmemFull[acc], accPhase, abortFlag)) { ok = false; break; }
            fenceAfterSync();
            const uint32_t taddr = tmemBase + acc * kBlockN + ((quarter * 32u) << 16);
            uint32_t* counter = p.splitCounters + (w.tile * 2 + rank);
            if (w.kind == kWorkPartial)
            {
                publishPartial(p, taddr, p.splitWorkspace + clusterId * slotStride + (rank * 128 + rowInCta) * size_t(256));
                fenceBeforeSync();
                mbarArriveCluster(leaderEmpty + acc * 8);
                __threadfence();
                epilogueBarrier();
                if (captain) atomicAdd(counter, 1u);
            }
            else
            {
                if (captain)
                {
                    const uint64_t start = globalTimerNs();
                    uint32_t seen = 0, spins = 0;
                    for (;;)
                    {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                        if (seen >= w.partials) break;
                        if ((++spins & 63u) == 0)
                        {
                            if (*abortFlag) break;
                            if (globalTimerNs() - start > kWaitLimitNs) { *abortFlag = 1; break; }
                        }
                    }
                    __threadfence();
                }
                epilogueBarrier();
                if (*abortFlag) { ok = false; break; }
                finishTile(p, taddr, row, tn * p.blockN,
                           p.splitWorkspace + (clusterId + 1) * slotStride + (rank * 128 + rowInCta) * size_t(256), slotStride, w.partials);
                fenceBeforeSync();
                mbarArriveCluster(leaderEmpty + acc * 8);
                if (captain) *counter = 0;            // every partial of this tile has arrived: ready for the next launch
            }
            acc ^= 1u;
            if (acc == 0) accPhase ^= 1u;
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // staging buffers are read, C is written
        }
    }

    if (threadIdx.x == 0) lingerAfterAbort(abortFlag);
    fenceBeforeSync();
    __syncthreads();
    clusterSync();                      // the leader's MMAs read the peer's shared memory until the very end
    if (warp == 1)
    {
        fenceAfterSync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(kTmemColumns) : "memory");
    }
    if (threadIdx.x == 0 && s.abortFlag) atomicExch(p.errorWord, 1u);
}

// ---- f32 split pass: src (any 2-D strides) -> K-major scratch, zero padded to kPad (a multiple of 64) ---------------
//   hi32[rows][kPad]      a rounded to TF32 (low 13 mantissa bits zero): operand of the main pass
//   pair16[rows][2*kPad]  [ bf16(a) | bf16(a - hi) ]: operands of the two cross-term passes
// One CTA converts a 64 x 64 tile; every thread owns runs of 8 consecutive k, so that all three outputs leave as
// 16-byte stores (12 bytes written per 4 bytes read: the pass is bound by HBM writes). A source whose unit stride runs
// along k is read in place with 16-byte loads; one whose unit stride runs along the rows is read with 16-byte loads
// along the rows and turned through shared memory.
__device__ __forceinline__ void splitEmit(const float (&v)[8], uint32_t r, uint32_t c, uint32_t kPad, float* __restrict__ hi32, uint16_t* __restrict__ pair16)
{
    float hi[8];
    uint32_t full[4], low[4];
    #pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const uint32_t bits = __float_as_uint(v[j]);
        // round to nearest even at 10 mantissa bits; values that would overflow keep their truncated form
        uint32_t rounded = (bits + 0xFFFu + ((bits >> 13) & 1u)) & 0xFFFFE000u;
        if ((rounded & 0x7F800000u) == 0x7F800000u) rounded = bits & 0xFFFFE000u;
        hi[j] = __uint_as_float(rounded);
    }
    #pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        full[j] = static_cast<uint32_t>(dev::f32ToBf16(v[2 * j])) | (static_cast<uint32_t>(dev::f32ToBf16(v[2 * j + 1])) << 16);
        low[j] = static_cast<uint32_t>(dev::f32ToBf16(v[2 * j] - hi[2 * j])) | (static_cast<uint32_t>(dev::f32ToBf16(v[2 * j + 1] - hi[2 * j + 1])) << 16);
    }
    float4* h = reinterpret_cast<float4*>(hi32 + static_cast<uint64_t>(r) * kPad + c);
    h[0] = make_float4(hi[0], hi[1], hi[2], hi[3]);
    h[1] = make_float4(hi[4], hi[5], hi[6], hi[7]);
    uint16_t* out = pair16 + static_cast<uint64_t>(r) * (2ull * kPad) + c;
    *reinterpret_cast<uint4*>(out) = make_uint4(full[0], full[1], full[2], full[3]);
    *reinterpret_cast<uint4*>(out + kPad) = make_uint4(low[0], low[1], low[2], low[3]);
}

template <bool Transposed>
__global__ void __launch_bounds__(256) splitF32Kernel(const float* __restrict__ src, uint64_t rowStride, uint64_t colStride,
                                                      uint32_t rows, uint32_t k, uint32_t kPad, float* __restrict__ hi32,
                                                      uint16_t* __restrict__ pair16, uint32_t vectorLoads)
{
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    if (!Transposed)
    {
        #pragma unroll
        for (uint32_t it = 0; it < 2; ++it)
        {
            const uint32_t idx = threadIdx.x + it * 256;
            const uint32_t r = r0 + (idx >> 3), c = c0 + (idx & 7u) * 8;
            if (r >= rows) continue;
            float v[8];
            const float* in = src + static_cast<uint64_t>(r) * rowStride + static_cast<uint64_t>(c) * colStride;
            if (vectorLoads && c + 8 <= k)
            {
                const float4 x = reinterpret_cast<const float4*>(in)[0], y = reinterpret_cast<const float4*>(in)[1];
                v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
            }
            else
            {
                #pragma unroll
                for (uint32_t j = 0; j < 8; ++j) v[j] = (c + j < k) ? in[j * colStride] : 0.f;
            }
            splitEmit(v, r, c, kPad, hi32, pair16);
        }
    }
    else
    {
        __shared__ float tile[64][65];                        // [row][k]; odd pitch: both phases at most 2-way conflicts
        #pragma unroll
        for (uint32_t it = 0; it < 4; ++it)
        {
            const uint32_t idx = threadIdx.x + it * 256;
            const uint32_t kk = idx >> 4, rg = (idx & 15u) * 4;
            const uint32_t c = c0 + kk, r = r0 + rg;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < k)
            {
                const float* in = src + static_cast<uint64_t>(r) * rowStride + static_cast<uint64_t>(c) * colStride;
                if (vectorLoads && r + 4 <= rows) x = *reinterpret_cast<const float4*>(in);
                else
                {
                    if (r < rows) x.x = in[0];
                    if (r + 1 < rows) x.y = in[rowStride];
                    if (r + 2 < rows) x.z = in[2 * rowStride];
                    if (r + 3 < rows) x.w = in[3 * rowStride];
                }
            }
            tile[rg][kk] = x.x; tile[rg + 1][kk] = x.y; tile[rg + 2][kk] = x.z; tile[rg + 3][kk] = x.w;
        }
        __syncthreads();
        // same thread-to-output mapping as the in-place variant: 8 threads cover one row's 64 k, so the three output
        // streams leave as 256- and 128-byte runs per row
        #pragma unroll
        for (uint32_t it = 0; it < 2; ++it)
        {
            const uint32_t idx = threadIdx.x + it * 256;
            const uint32_t r = idx >> 3, kg = (idx & 7u) * 8;
            if (r0 + r >= rows) continue;
            float v[8];
            #pragma unroll
            for (uint32_t j = 0; j < 8; ++j) v[j] = tile[r][kg + j];
            splitEmit(v, r0 + r, c0 + kg, kPad, hi32, pair16);
        }
    }
}

// ---- half-term scheme: max|x| of a strided 2-D operand, then the scaled two-term fp16 split ---------------------------
// slot: bit pattern of the running maximum (non-negative floats order like unsigned integers), zeroed by the launcher.
__global__ void __launch_bounds__(256) absMaxKernel(const float* __restrict__ src, uint64_t outer, uint64_t inner, uint64_t outerStride,
                                                    uint64_t innerStride, uint32_t vectorLoads, uint32_t* slot)
{
    uint32_t best = 0;
    if (vectorLoads && outerStride == inner) { inner *= outer; outerStride = inner; outer = 1; }    // dense: one long row, no divisions
    const uint64_t perRow = vectorLoads ? inner / 4 : inner;
    const uint64_t total = outer * perRow;
    const uint64_t threads = static_cast<uint64_t>(gridDim.x) * 256;
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    auto fold4 = [&](const float4& x)
    {
        best = max(max(best, __float_as_uint(fabsf(x.x))), max(__float_as_uint(fabsf(x.y)), max(__float_as_uint(fabsf(x.z)), __float_as_uint(fabsf(x.w)))));
    };
    auto pack = [&](uint64_t idx)
    {
        if (outer == 1) return reinterpret_cast<const float4*>(src) + idx;
        const uint64_t o = idx / perRow, c = idx - o * perRow;
        return reinterpret_cast<const float4*>(src + o * outerStride + c * 4);
    };
    if (vectorLoads)
    {
        for (; i + 7 * threads < total; i += 8 * threads)          // eight independent 128-bit loads per thread
        {
            const float4 x0 = *pack(i), x1 = *pack(i + threads), x2 = *pack(i + 2 * threads), x3 = *pack(i + 3 * threads);
            const float4 x4 = *pack(i + 4 * threads), x5 = *pack(i + 5 * threads), x6 = *pack(i + 6 * threads), x7 = *pack(i + 7 * threads);
            fold4(x0); fold4(x1); fold4(x2); fold4(x3); fold4(x4); fold4(x5); fold4(x6); fold4(x7);
        }
        for (; i < total; i += threads) fold4(*pack(i));
    }
    else
    {
        for (; i < total; i += threads)
        {
            const uint64_t o = i / perRow, c = i - o * perRow;
            best = max(best, __float_as_uint(fabsf(src[o * outerStride + c * innerStride])));
        }
    }
    // NaNs carry the largest patterns: a NaN anywhere ends up as the maximum and switches the scaling off
    #pragma unroll
    for (int d = 16; d > 0; d >>= 1) best = max(best, __shfl_down_sync(0xffffffffu, best, d));
    __shared__ uint32_t warpBest[8];
    if ((threadIdx.x & 31) == 0) warpBest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0)                                   // one atomic per CTA: they all hit the same word
    {
        #pragma unroll
        for (int w = 1; w < 8; ++w) best = max(best, warpBest[w]);
        if (best != 0) atomicMax(slot, best);
    }
}

//   terms[rows][2*kPad]  [ h0 | h1 ] with h0 = fp16(s*a), h1 = fp16(s*a - h0), s = halfTermScale(max|a|):  s*a = h0 + h1 to 22 bits
__device__ __forceinline__ void splitEmitHalf(const float (&v)[8], float scale, uint32_t r, uint32_t c, uint32_t kPad, uint32_t outPitch, uint16_t* __restrict__ terms)
{
    uint32_t h0[4], h1[4];
    #pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        const float x0 = v[2 * j] * scale, x1 = v[2 * j + 1] * scale;
        const uint16_t a0 = dev::f32ToF16(x0), a1 = dev::f32ToF16(x1);
        h0[j] = static_cast<uint32_t>(a0) | (static_cast<uint32_t>(a1) << 16);
        h1[j] = static_cast<uint32_t>(dev::f32ToF16(x0 - dev::f16ToF32(a0))) | (static_cast<uint32_t>(dev::f32ToF16(x1 - dev::f16ToF32(a1))) << 16);
    }
    uint16_t* out = terms + static_cast<uint64_t>(r) * outPitch + c;
    *reinterpret_cast<uint4*>(out) = make_uint4(h0[0], h0[1], h0[2], h0[3]);
    *reinterpret_cast<uint4*>(out + kPad) = make_uint4(h1[0], h1[1], h1[2], h1[3]);
}

template <bool Transposed>
__global__ void __launch_bounds__(256) splitF16Kernel(const float* __restrict__ src, uint64_t rowStride, uint64_t colStride, uint32_t rows,
                                                      uint32_t k, uint32_t kPad, uint32_t outPitch, uint16_t* __restrict__ terms, uint32_t vectorLoads,
                                                      const uint32_t* __restrict__ maxBits)
{
    const float scale = halfTermScale(*maxBits);
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    if (!Transposed)
    {
        #pragma unroll
        for (uint32_t it = 0; it < 2; ++it)
        {
            const uint32_t idx = threadIdx.x + it * 256;
            const uint32_t r = r0 + (idx >> 3), c = c0 + (idx & 7u) * 8;
            if (r >= rows) continue;
            float v[8];
            const float* in = src + static_cast<uint64_t>(r) * rowStride + static_cast<uint64_t>(c) * colStride;
            if (vectorLoads && c + 8 <= k)
            {
                const float4 x = reinterpret_cast<const float4*>(in)[0], y = reinterpret_cast<const float4*>(in)[1];
                v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
            }
            else
            {
                #pragma unroll
                for (uint32_t j = 0; j < 8; ++j) v[j] = (c + j < k) ? in[j * colStride] : 0.f;
            }
            splitEmitHalf(v, scale, r, c, kPad, outPitch, terms);
        }
    }
    else
    {
        __shared__ float tile[64][65];                        // [row][k]
        #pragma unroll
        for (uint32_t it = 0; it < 4; ++it)
        {
            const uint32_t idx = threadIdx.x + it * 256;
            const uint32_t kk = idx >> 4, rg = (idx & 15u) * 4;
            const uint32_t c = c0 + kk, r = r0 + rg;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < k)
            {
                const float* in = src + static_cast<uint64_t>(r) * rowStride + static_cast<uint64_t>(c) * colStride;
                if (vectorLoads && r + 4 <= rows) x = *reinterpret_cast<const float4*>(in);
                else
                {
                    if (r < rows) x.x = in[0];
                    if (r + 1 < rows) x.y = in[rowStride];
                    if (r + 2 < rows) x.z = in[2 * rowStride];
                    if (r + 3 < rows) x.w = in[3 * rowStride];
                }
            }
            tile[rg][kk] = x.x; tile[rg + 1][kk] = x.y; tile[rg + 2][kk] = x.z; tile[rg + 3][kk] = x.w;
        }
        __syncthreads();
        #pragma unroll
        for (uint32_t it = 0; it < 2; ++it)
        {
            const uint32_t idx = threadIdx.x + it * 256;
            const uint32_t r = idx >> 3, kg = (idx & 7u) * 8;
            if (r0 + r >= rows) continue;
            float v[8];
            #pragma unroll
            for (uint32_t j = 0; j < 8; ++j) v[j] = tile[r][kg + j];
            splitEmitHalf(v, scale, r0 + r, c0 + kg, kPad, outPitch, terms);
        }
    }
}

// max|x| of the operand into *slot (zeroed beforehand), then its two-term fp16 split.
void launchHalfTermSplit(cudaStream_t stream, int smCount, const float* src, uint64_t rowStride, uint64_t colStride, uint32_t rows, uint32_t k,
                         uint32_t kPad, uint32_t outPitch, uint16_t* terms, uint32_t* slot, bool maxKnown = false)
{
    const bool aligned = reinterpret_cast<uintptr_t>(src) % 16 == 0;
    const unsigned maxGrid = static_cast<unsigned>(smCount) * 8;
    if (colStride == 1 || rowStride != 1)
    {
        const uint32_t vec = colStride == 1 && aligned && rowStride % 4 == 0 && k % 4 == 0;
        const uint64_t items = static_cast<uint64_t>(rows) * (vec ? k / 4 : k);
        if (!maxKnown)
            absMaxKernel<<<static_cast<unsigned>(std::min<uint64_t>(maxGrid, (items + 255) / 256)), 256, 0, stream>>>(src, rows, k, rowStride, colStride, vec, slot);
        splitF16Kernel<false><<<dim3(kPad / 64, (rows + 63) / 64), 256, 0, stream>>>(src, rowStride, colStride, rows, k, kPad, outPitch, terms,
                                                                                      colStride == 1 && aligned && rowStride % 4 == 0, slot);
    }
    else
    {
        const uint32_t vec = aligned && colStride % 4 == 0 && rows % 4 == 0;
        const uint64_t items = static_cast<uint64_t>(k) * (vec ? rows / 4 : rows);
        if (!maxKnown)
            absMaxKernel<<<static_cast<unsigned>(std::min<uint64_t>(maxGrid, (items + 255) / 256)), 256, 0, stream>>>(src, k, rows, colStride, rowStride, vec, slot);
        splitF16Kernel<true><<<dim3(kPad / 64, (rows + 63) / 64), 256, 0, stream>>>(src, rowStride, colStride, rows, k, kPad, outPitch, terms,
                                                                                     aligned && colStride % 4 == 0, slot);
    }
}

// Launches the split of a rows x k operand whose element (r, c) sits at src[r * rowStride + c * colStride].
void launchSplit(cudaStream_t stream, const float* src, uint64_t rowStride, uint64_t colStride, uint32_t rows, uint32_t k, uint32_t kPad,
                 float* hi32, uint16_t* pair16)
{
    const dim3 grid(kPad / 64, (rows + 63) / 64);
    const bool aligned = reinterpret_cast<uintptr_t>(src) % 16 == 0;
    if (colStride == 1 || rowStride != 1)
    {
        // unit stride along k (or no unit stride at all: element loads)
        const uint32_t vec = colStride == 1 && aligned && rowStride % 4 == 0;
        splitF32Kernel<false><<<grid, 256, 0, stream>>>(src, rowStride, colStride, rows, k, kPad, hi32, pair16, vec);
    }
    else
    {
        const uint32_t vec = aligned && colStride % 4 == 0;
        splitF32Kernel<true><<<grid, 256, 0, stream>>>(src, rowStride, colStride, rows, k, kPad, hi32, pair16, vec);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeTiled()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []
    {
        cudaDriverEntryPointQueryResult status;
        void* p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) == cudaSuccess && status == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D tensor map over a matrix whose fast dimension has `inner` elements and whose rows are `pitchBytes` apart.
bool makeMap(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t outer, uint64_t pitchBytes,
             uint32_t boxInner, uint32_t boxOuter)
{
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitchBytes};
    cuuint32_t box[2] = {boxInner, boxOuter};
    cuuint32_t elemStrides[2] = {1, 1};
    EncodeTiledFn fn = encodeTiled();
    if (!fn) return false;
    return fn(map, type, 2, const_cast<void*>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D view of an MN-major matrix (mn fastest): (64 mn, k, mn / 64). One box {64, boxK, atoms} lands in shared memory
// as `atoms` consecutive 64-mn x boxK blocks - the layout the MN-major descriptors expect - with one TMA instruction.
bool makeMap3d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t mn, uint64_t k, uint64_t pitchBytes, uint32_t boxK,
               uint32_t atoms)
{
    cuuint64_t dims[3] = {64, k, mn / 64};
    cuuint64_t strides[2] = {pitchBytes, 128};
    cuuint32_t box[3] = {64, boxK, atoms};
    cuuint32_t elemStrides[3] = {1, 1, 1};
    EncodeTiledFn fn = encodeTiled();
    if (!fn) return false;
    return fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D view of a K-major matrix (k fastest): (atomElems k, rows, k / atomElems), atomElems = 128 bytes of K. One box
// {atomElems, boxRows, 2} lands as two consecutive K-major swizzle atoms of boxRows rows: 256 contiguous bytes per row.
bool makeMapK3d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t rows, uint64_t kElems, uint64_t pitchBytes,
                uint32_t atomElems, uint32_t boxRows)
{
    cuuint64_t dims[3] = {atomElems, rows, kElems / atomElems};
    cuuint64_t strides[2] = {pitchBytes, 128};
    cuuint32_t box[3] = {atomElems, boxRows, 2};
    cuuint32_t elemStrides[3] = {1, 1, 1};
    EncodeTiledFn fn = encodeTiled();
    if (!fn) return false;
    return fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Operand
{
    const void* base;
    bool        mnMajor;       // unit stride runs along M (for A) or N (for B) instead of K
    uint64_t    pitch;         // elements between consecutive lines of the slow dimension
};

// Classifies a strided 2-D operand (rows x cols, the K dimension being `kIsCols ? cols : rows`).
bool classify(const void* base, uint64_t rowStride, uint64_t colStride, uint64_t rows, uint64_t cols, bool kIsCols, size_t esize, Operand* out)
{
    const bool colsContiguous = colStride == 1 || cols == 1;
    const bool rowsContiguous = rowStride == 1 || rows == 1;
    if (colsContiguous && (rows == 1 || rowStride >= cols))
    {
        out->base = base; out->pitch = rows == 1 ? cols : rowStride; out->mnMajor = !kIsCols;
    }
    else if (rowsContiguous && (cols == 1 || colStride >= rows))
    {
        out->base = base; out->pitch = cols == 1 ? rows : colStride; out->mnMajor = kIsCols;
    }
    else return false;
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (out->pitch * esize) % 16 != 0) return false;
    return true;
}

}   // namespace

namespace
{
// The give-up path of mbarWait on its own: thread 0 waits for a phase that never completes, the wait runs out after
// limitNs, and the kernel reports it the way the matmul kernels do. The limit is capped so that a wrong argument cannot
// park the kernel for long.
__global__ void boundedWaitSelfTestKernel(uint64_t limitNs, uint32_t* errorWord)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abortFlag;
    if (threadIdx.x == 0)
    {
        mbarInit(&bar, 1);
        abortFlag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        const uint64_t limit = limitNs < 100000000ull ? limitNs : 100000000ull;
        mbarWait(&bar, 0, &abortFlag, limit);           // nobody arrives: returns false once the limit has passed
    }
    __syncthreads();
    if (threadIdx.x == 0 && abortFlag) atomicExch(errorWord, 1u);
}
}   // namespace

void launchBoundedWaitSelfTest(const kernels::LaunchContext& ctx, uint64_t limitNs)
{
    boundedWaitSelfTestKernel<<<1, 32, 0, ctx.stream>>>(limitNs, reinterpret_cast<uint32_t*>(static_cast<char*>(ctx.scratch) + kernels::kScratchTimeoutOffset));
    if (ctx.launches) ++*ctx.launches;
}

// The conditions under which launchTensorCore takes the three-fp16-pass CTA-pair kernel with TMA stores - the one whose
// epilogue can fold a bias add and a tanh. Kept in step with the choices made there.
bool canFoldEpilogue(const Problem& q, bool needDriver)
{
    static const bool enabled = []{ const char* v = std::getenv("AIXB200_GEMM_EPILOGUE"); return !(v && v[0] == '0'); }();
    static const bool tensorCoreOff = std::getenv("AIXB200_NO_TENSOR_CORE") != nullptr;
    static const bool pairEnabled = []{ const char* v = std::getenv("AIXB200_GEMM_PAIR"); return !(v && v[0] == '0'); }();
    static const bool halfTerms = []{ const char* v = std::getenv("AIXB200_GEMM_F32"); return !(v && v[0] == 'h' && v[1] == 'y'); }();
    static const bool tmaStoreEnabled = []{ const char* v = std::getenv("AIXB200_GEMM_TMA_STORE"); return !(v && v[0] == '0'); }();
    if (!enabled || tensorCoreOff || !pairEnabled || !halfTerms || !tmaStoreEnabled) return false;
    if (q.dtype != F32 || !q.splitF32) return false;
    if (q.m <= 128 || q.n < 64 || q.k < 32) return false;
    if (q.m > 0x7FFFFF00ull || q.n > 0x7FFFFF00ull || q.k > 0x3FFFFF00ull) return false;
    if ((q.n * 4) % 16 != 0) return false;
    for (const void* ptr : {static_cast<const void*>(q.c), static_cast<const void*>(q.bias), static_cast<const void*>(q.biasOut), static_cast<const void*>(q.tanhOut)})
        if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return false;
    return !needDriver || encodeTiled() != nullptr;
}

bool launchTensorCore(Device& device, const kernels::LaunchContext& ctx, const Problem& q)
{
    if (q.dtype != F32 && q.dtype != BF16 && q.dtype != F16) return false;
    if (q.dtype == F32 && !q.splitF32) return false;
    if (q.m < 64 || q.n < 64 || q.k < 32) return false;                     // tiny problems: launch-bound, CUDA cores do
    if (q.m > 0x7FFFFF00ull || q.n > 0x7FFFFF00ull || q.k > 0x3FFFFF00ull) return false;
    if (!encodeTiled()) return false;
    static bool disabled = std::getenv("AIXB200_NO_TENSOR_CORE") != nullptr;
    if (disabled) return false;

    // CTA pairs (256 x 256 tiles) unless switched off or the problem has a single row of 128-row tiles.
    static const bool pairEnabled = []{ const char* v = std::getenv("AIXB200_GEMM_PAIR"); return !(v && v[0] == '0'); }();
    const bool pair = pairEnabled && q.m > 128;
    if (q.bias && !canFoldEpilogue(q, true)) return false;
    KernelParams p{};
    p.m = static_cast<uint32_t>(q.m); p.n = static_cast<uint32_t>(q.n); p.k = static_cast<uint32_t>(q.k);
    p.tilesM = pair ? (p.m + 255) / 256 : (p.m + kBlockM - 1) / kBlockM;
    // Tile width: 256 columns keep the tensor pipe busiest (measured: a 128-column tile reaches about 0.62 of its
    // throughput), but a persistent grid loses the idle part of its last wave of tiles; narrow tiles only pay off
    // when that loss is larger still (few tiles). Pick by the modelled efficiency.
    {
        const double workers = pair ? ctx.smCount / 2 : ctx.smCount;
        auto efficiency = [&](uint32_t blockN, double perTile)
        {
            const double tiles = static_cast<double>(p.tilesM) * ((p.n + blockN - 1) / blockN);
            // 16-bit problems on CTA pairs share the remainder wave along K (see WorkIterator): no idle tail to model
            static const bool splitOn = []{ const char* v = std::getenv("AIXB200_GEMM_SPLITK"); return v && v[0] == '1'; }();
            const bool sharedTail = splitOn && pair && q.dtype != F32 && (q.k + 63) / 64 >= 8 && tiles * ((q.k + 63) / 64) >= workers;
            const double waves = sharedTail ? std::max(1.0, tiles / workers) : std::ceil(tiles / workers);
            return perTile * tiles / (waves * workers) * (static_cast<double>(p.n) / (((p.n + blockN - 1) / blockN) * blockN));
        };
        static const int forced = []{ const char* v = std::getenv("AIXB200_GEMM_BLOCKN"); return v ? std::atoi(v) : 0; }();
        p.blockN = (forced == 128 || forced == 256) ? static_cast<uint32_t>(forced) : (efficiency(128, 0.62) > efficiency(256, 1.0) ? 128u : 256u);
    }
    p.tilesN = (p.n + p.blockN - 1) / p.blockN;
    {
        static const int group = []{ const char* v = std::getenv("AIXB200_GEMM_GROUP"); return v ? std::atoi(v) : 0; }();
        p.tileGroup = group > 0 ? static_cast<uint32_t>(group) : 16u;      // measured: 16 >= 8 > 4 > 2 by 1-2 % at 4096^3 and 8192^3
    }
    const uint32_t bRows = pair ? p.blockN / 2 : p.blockN;                   // B rows (N) each CTA loads per stage
    p.c = q.c;
    p.outDtype = q.dtype;
    p.vectorStores = (reinterpret_cast<uintptr_t>(q.c) % 16 == 0) && ((q.n * dtypeSize(q.dtype)) % 16 == 0);
    p.errorWord = reinterpret_cast<uint32_t*>(static_cast<char*>(ctx.scratch) + 128);
    CUtensorMap mapA, mapB, mapA16, mapB16;
    const bool tf32 = q.dtype == F32;

    if (!tf32)
    {
        Operand a, b;
        static const bool box3d = []{ const char* v = std::getenv("AIXB200_GEMM_BOX3D"); return !(v && v[0] == '0'); }();
        if (!classify(q.a, q.aRowStride, q.aColStride, q.m, q.k, true, 2, &a)) return false;
        if (!classify(q.b, q.bRowStride, q.bColStride, q.k, q.n, false, 2, &b)) return false;
        p.blockK = 64;
        p.kBlocks = (p.k + 63) / 64;
        p.kPhases = 1;
        p.chunkBlocks = p.kBlocks;
        p.chunks = 1;
        p.mmasPerStage = 4;
        const CUtensorMapDataType type = q.dtype == BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        p.aMnMajor = a.mnMajor; p.bMnMajor = b.mnMajor;
        if (!pair)
        {
            if (a.mnMajor)
            {
                p.aBoxes = kBlockM / 64; p.aBoxBytes = 64 * 128; p.aBoxStepMn = 64; p.aLbo = 64 * 128; p.kAdvanceA = 16 * 128;
                if (!makeMap(&mapA, type, a.base, q.m, q.k, a.pitch * 2, 64, 64)) return false;
            }
            else
            {
                p.aBoxes = 1; p.aBoxBytes = kStageBytesA; p.aLbo = 0; p.kAdvanceA = 32;
                if (!makeMap(&mapA, type, a.base, q.k, q.m, a.pitch * 2, 64, kBlockM)) return false;
            }
            if (b.mnMajor)
            {
                p.bBoxes = bRows / 64; p.bBoxBytes = 64 * 128; p.bBoxStepMn = 64; p.bLbo = 64 * 128; p.kAdvanceB = 16 * 128;
                if (!makeMap(&mapB, type, b.base, q.n, q.k, b.pitch * 2, 64, 64)) return false;
            }
            else
            {
                p.bBoxes = 1; p.bBoxBytes = bRows * 128; p.bLbo = 0; p.kAdvanceB = 32;
                if (!makeMap(&mapB, type, b.base, q.k, q.n, b.pitch * 2, 64, bRows)) return false;
            }
        }
        else
        {
            // stages of 128 elements of K: two swizzle atoms per operand
            p.atomK = 64;
            p.kBlocks = (p.k + 127) / 128;
            p.chunkBlocks = p.kBlocks;
            auto plan = [&](const Operand& op, uint64_t mn, uint32_t rows, CUtensorMap* map, uint32_t* load3d, uint32_t* bytes, uint32_t* lbo, uint32_t* off)
            {
                if (op.mnMajor)
                {
                    const uint32_t atoms = rows / 64;
                    *bytes = atoms * 128 * 128; *lbo = 128 * 128;
                    for (uint32_t j = 0; j < 8; ++j) off[j] = (j * 16 * 128) >> 4;
                    *load3d = box3d && mn % 64 == 0;
                    return *load3d ? makeMap3d(map, type, op.base, mn, q.k, op.pitch * 2, 128, atoms) : makeMap(map, type, op.base, mn, q.k, op.pitch * 2, 64, 64);
                }
                *bytes = rows * 256; *lbo = 0;
                for (uint32_t j = 0; j < 8; ++j) off[j] = ((j / 4) * rows * 128 + (j % 4) * 32) >> 4;
                *load3d = box3d && q.k % 64 == 0;
                return *load3d ? makeMapK3d(map, type, op.base, mn, q.k, op.pitch * 2, 64, rows) : makeMap(map, type, op.base, q.k, mn, op.pitch * 2, 64, rows);
            };
            if (!plan(a, q.m, kBlockM, &mapA, &p.aLoad3d, &p.pairABytes, &p.pairALbo, p.pairAOff)) return false;
            if (!plan(b, q.n, bRows, &mapB, &p.bLoad3d, &p.pairBBytes, &p.pairBLbo, p.pairBOff)) return false;
        }
        mapA16 = mapA; mapB16 = mapB;                      // unused by 16-bit problems
        // instruction descriptor: D = f32, A/B = bf16 or f16, majors, N >> 3, M >> 4
        p.idesc = (1u << 4) | ((q.dtype == BF16 ? 1u : 0u) << 7) | ((q.dtype == BF16 ? 1u : 0u) << 10) |
                  ((a.mnMajor ? 1u : 0u) << 15) | ((b.mnMajor ? 1u : 0u) << 16) | ((p.blockN >> 3) << 17) | (((pair ? 256u : 128u) >> 4) << 24);
    }
    else
    {
        // Split into K-major scratch (see splitF32Kernel). kPad is a multiple of 64 so that bf16 stages (64 elements)
        // and TF32 stages (32 elements) cover the same K ranges.
        const uint32_t kPad = (p.k + 127) & ~127u;
        p.kPhases = 3;
        p.kPerPhase = kPad;
        p.aPlane = p.bPlane = kPad;
        // Pair kernel: three fp16 passes over scaled two-term operands (AIXB200_GEMM_F32=hybrid: TF32 + bf16 cross terms).
        static const bool halfTerms = []{ const char* v = std::getenv("AIXB200_GEMM_F32"); return !(v && v[0] == 'h' && v[1] == 'y'); }();
        if (pair && halfTerms)
        {
            // Every operand as two scaled fp16 terms. A tensor that is dense along one of its two dimensions is prepared
            // ONCE, in its own row-major layout [rows][h0 | h1] (Device::PreparedTerms), and read K-major or MN-major
            // through the matching tensor map and descriptors: the forward product, dX and dW then share one prepared
            // form of every activation, weight and gradient instead of splitting each of them once per orientation.
            // Operands with two non-unit strides are split into a temporary K-major buffer for this call only.
            struct Prepared { const uint16_t* terms; const uint32_t* scale; bool mnMajor; uint32_t plane; };
            uint32_t* tempSlots = reinterpret_cast<uint32_t*>(static_cast<char*>(ctx.scratch) + ctx.scratchBytes + 2048);   // behind the split-tile counters
            uint64_t preparedLaunches = 0;
            auto prepare = [&](const void* base, uint64_t mnStride, uint64_t kStride, uint64_t mn, uint32_t boxRows, uint32_t* tempSlot,
                               CUtensorMap* map, Prepared* out) -> bool
            {
                const float* src = static_cast<const float*>(base);
                const bool kDense = (kStride == 1 || p.k == 1) && (mn == 1 || mnStride >= p.k);
                const bool mnDense = (mnStride == 1 || mn == 1) && (p.k == 1 || kStride >= mn);
                // only tensors of this device's allocator: writes into foreign memory cannot be seen, so nothing is kept of it
                if (device.preparedTermsEnabled() && (kDense || mnDense) && device.ownsMemory(base))
                {
                    const uint64_t rows = kDense ? mn : p.k, cols = kDense ? p.k : mn;
                    const uint64_t pitch = rows == 1 ? cols : (kDense ? mnStride : kStride);
                    const Device::PreparedTerms* e = device.findPreparedTerms(base, rows, cols, pitch);
                    if (!e)
                    {
                        e = device.addPreparedTerms(base, rows, cols, pitch);
                        // the kernel that wrote the tensor may have left max|x| in the slot already (e->ownsSlot == false)
                        if (e->ownsSlot && cudaMemsetAsync(device.preparedSlot(e->slot), 0, 4, ctx.stream) != cudaSuccess) return false;
                        launchHalfTermSplit(ctx.stream, ctx.smCount, src, pitch, 1, static_cast<uint32_t>(rows), static_cast<uint32_t>(cols),
                                            static_cast<uint32_t>(e->paddedCols), static_cast<uint32_t>(e->termPitch), static_cast<uint16_t*>(e->terms),
                                            device.preparedSlot(e->slot), !e->ownsSlot);
                        preparedLaunches += e->ownsSlot ? 2 : 1;
                    }
                    out->terms = static_cast<const uint16_t*>(e->terms);
                    out->scale = device.preparedSlot(e->slot);
                    out->mnMajor = !kDense;
                    out->plane = static_cast<uint32_t>(e->paddedCols);
                    const uint64_t rowBytes = e->termPitch * 2;
                    return kDense ? makeMapK3d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, e->terms, mn, 2ull * e->paddedCols, rowBytes, 64, boxRows)
                                  : makeMap3d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, e->terms, 2ull * e->paddedCols, p.k, rowBytes, 128, boxRows / 64);
                }
                uint16_t* terms = static_cast<uint16_t*>(device.temporary(static_cast<size_t>(mn) * 2 * kPad * 2));
                if (cudaMemsetAsync(tempSlot, 0, 4, ctx.stream) != cudaSuccess) return false;
                launchHalfTermSplit(ctx.stream, ctx.smCount, src, mnStride, kStride, static_cast<uint32_t>(mn), p.k, kPad, 2 * kPad, terms, tempSlot);
                preparedLaunches += 2;
                out->terms = terms; out->scale = tempSlot; out->mnMajor = false; out->plane = kPad;
                return makeMapK3d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, terms, mn, 2ull * kPad, 2ull * kPad * 2, 64, boxRows);
            };
            Prepared pa{}, pb{};
            if (!prepare(q.a, q.aRowStride, q.aColStride, q.m, kBlockM, tempSlots, &mapA16, &pa)) return false;
            // B is k x n: its M/N dimension are the n columns
            if (!prepare(q.b, q.bColStride, q.bRowStride, q.n, bRows, tempSlots + 1, &mapB16, &pb)) return false;
            if (ctx.launches) *ctx.launches += preparedLaunches;
            p.halfTerms = 1;
            p.scaleA = pa.scale; p.scaleB = pb.scale;
            p.aPlane = pa.plane; p.bPlane = pb.plane;
            p.aMnMajor = pa.mnMajor; p.bMnMajor = pb.mnMajor;
            p.atomK = 64;
            p.kBlocks = kPad / 128;                              // stages of 128 fp16 elements in all three passes
            {
                // 256 elements of K per in-TMEM partial sum: the tensor core's accumulation truncates, an error that grows with
                // the number of MMAs folded into one accumulator, and with the running sums kept in registers a short chunk
                // costs nothing (measured: 2, 4 and 96 stages per chunk run 4096^3 within 1 % of each other).
                // AIXB200_GEMM_HCHUNK: stages per partial sum, for measurements only - long chunks leave the f32 error bar.
                static const int chunkOverride = []{ const char* v = std::getenv("AIXB200_GEMM_HCHUNK"); return v ? std::atoi(v) : 0; }();
                p.chunkBlocks = chunkOverride > 0 ? static_cast<uint32_t>(chunkOverride) : 2u;
            }
            p.aLoad3d = p.bLoad3d = 1;
            p.pairABytes = kBlockM * 256; p.pairBBytes = bRows * 256;
            p.pairALbo = pa.mnMajor ? 128 * 128 : 0; p.pairBLbo = pb.mnMajor ? 128 * 128 : 0;
            for (uint32_t j = 0; j < 8; ++j)
            {
                p.pairAOff[j] = pa.mnMajor ? (j * 16 * 128) >> 4 : ((j / 4) * kBlockM * 128 + (j % 4) * 32) >> 4;
                p.pairBOff[j] = pb.mnMajor ? (j * 16 * 128) >> 4 : ((j / 4) * bRows * 128 + (j % 4) * 32) >> 4;
            }
            mapA = mapA16; mapB = mapB16;                        // no 32-bit pass
        }
        else
        {
        float* hiA = static_cast<float*>(device.temporary(static_cast<size_t>(p.m) * kPad * 4));
        float* hiB = static_cast<float*>(device.temporary(static_cast<size_t>(p.n) * kPad * 4));
        uint16_t* pairA = static_cast<uint16_t*>(device.temporary(static_cast<size_t>(p.m) * 2 * kPad * 2));
        uint16_t* pairB = static_cast<uint16_t*>(device.temporary(static_cast<size_t>(p.n) * 2 * kPad * 2));
        launchSplit(ctx.stream, static_cast<const float*>(q.a), q.aRowStride, q.aColStride, p.m, p.k, kPad, hiA, pairA);
        // B is k x n: its "rows" for the split are the n columns
        launchSplit(ctx.stream, static_cast<const float*>(q.b), q.bColStride, q.bRowStride, p.n, p.k, kPad, hiB, pairB);
        if (ctx.launches) *ctx.launches += 2;
        if (!pair)
        {
            p.blockK = 32;
            p.kBlocks = kPad / 32;
            p.chunkBlocks = 16;                                  // 512 elements of K per in-TMEM partial sum
            p.mmasPerStage = 4;
            p.aBoxes = 1; p.aBoxBytes = kStageBytesA; p.kAdvanceA = 32;
            p.bBoxes = 1; p.bBoxBytes = bRows * 128; p.kAdvanceB = 32;
            if (!makeMap(&mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, hiA, kPad, q.m, static_cast<uint64_t>(kPad) * 4, 32, kBlockM)) return false;
            if (!makeMap(&mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, hiB, kPad, q.n, static_cast<uint64_t>(kPad) * 4, 32, bRows)) return false;
            if (!makeMap(&mapA16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, pairA, 2ull * kPad, q.m, 2ull * kPad * 2, 64, kBlockM)) return false;
            if (!makeMap(&mapB16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, pairB, 2ull * kPad, q.n, 2ull * kPad * 2, 64, bRows)) return false;
        }
        else
        {
            // stages of 64 TF32 elements (main pass) or 128 bf16 elements (cross passes), all K-major, one 3-D box each
            p.atomK = 32;
            p.kBlocks = kPad / 64;
            // 512 elements of K per in-TMEM partial sum (AIXB200_GEMM_CHUNK: in stages of 64, even; for measurements)
            static const int chunkOverride = []{ const char* v = std::getenv("AIXB200_GEMM_CHUNK"); return v ? std::atoi(v) : 0; }();
            p.chunkBlocks = (chunkOverride >= 2 && chunkOverride % 2 == 0) ? static_cast<uint32_t>(chunkOverride) : 8u;
            p.aLoad3d = p.bLoad3d = 1;
            p.pairABytes = kBlockM * 256; p.pairBBytes = bRows * 256;
            for (uint32_t j = 0; j < 8; ++j)
            {
                p.pairAOff[j] = ((j / 4) * kBlockM * 128 + (j % 4) * 32) >> 4;
                p.pairBOff[j] = ((j / 4) * bRows * 128 + (j % 4) * 32) >> 4;
            }
            if (!makeMapK3d(&mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, hiA, q.m, kPad, static_cast<uint64_t>(kPad) * 4, 32, kBlockM)) return false;
            if (!makeMapK3d(&mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, hiB, q.n, kPad, static_cast<uint64_t>(kPad) * 4, 32, bRows)) return false;
            if (!makeMapK3d(&mapA16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, pairA, q.m, 2ull * kPad, 2ull * kPad * 2, 64, kBlockM)) return false;
            if (!makeMapK3d(&mapB16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, pairB, q.n, 2ull * kPad, 2ull * kPad * 2, 64, bRows)) return false;
        }
        }
        p.chunks = (p.kBlocks + p.chunkBlocks - 1) / p.chunkBlocks;
        const uint32_t shape = ((p.blockN >> 3) << 17) | (((pair ? 256u : 128u) >> 4) << 24);
        p.idesc = (1u << 4) | (2u << 7) | (2u << 10) | shape;            // D f32, A/B tf32
        p.idesc16 = p.halfTerms ? ((1u << 4) | ((p.aMnMajor ? 1u : 0u) << 15) | ((p.bMnMajor ? 1u : 0u) << 16) | shape)   // D f32, A/B f16
                                : ((1u << 4) | (1u << 7) | (1u << 10) | shape);   // D f32, A/B bf16
    }

    // The opt-in to more than 48 KiB of dynamic shared memory and the cluster occupancy are properties of one device:
    // kept per ordinal, so a second device handle on another GPU of the same process sets them up for itself.
    constexpr int kMaxDevices = 64;
    struct PerDevice { std::mutex lock; bool attributesSet = false; int maxClusters = 0; };
    static PerDevice perDevice[kMaxDevices];
    const int ordinal = device.ordinal();
    if (ordinal < 0 || ordinal >= kMaxDevices) return false;
    PerDevice& state = perDevice[ordinal];
    const size_t smemBytes = sizeof(SharedStorage) + 1024;
    const size_t pairSmem = sizeof(PairStorage) + 1024;
    {
        std::lock_guard<std::mutex> guard(state.lock);
        if (!state.attributesSet)
        {
            cudaFuncSetAttribute(gemmKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes));
            cudaFuncSetAttribute(gemmKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes));
            cudaFuncSetAttribute(gemmPairKernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairSmem));
            cudaFuncSetAttribute(gemmPairKernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairSmem));
            cudaFuncSetAttribute(gemmPairKernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairSmem));
            cudaFuncSetAttribute(gemmPairKernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairSmem));
            cudaFuncSetAttribute(gemmPairKernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pairSmem));
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(static_cast<unsigned>(ctx.smCount) & ~1u);
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = pairSmem;
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&state.maxClusters, gemmPairKernel<0>, &cfg) != cudaSuccess || state.maxClusters <= 0)
            {
                cudaGetLastError();
                state.maxClusters = ctx.smCount / 2;
            }
            state.attributesSet = true;
        }
    }
    const int maxClusters = state.maxClusters;
    const uint32_t tiles = p.tilesM * p.tilesN;
    if (pair)
    {
        // A collective on the device's side stream needs SMs of its own. The persistent grid would otherwise either keep
        // it out until the matmul ends or, if the collective got there first, start some of its clusters late - and
        // with tiles dealt out statically those late clusters finish their whole share late. While a collective is in
        // flight the grid can therefore leave a few SMs free (AIXB200_GEMM_RESERVE_SMS; default 0 = off until measured).
        uint32_t usable = static_cast<uint32_t>(maxClusters);
        if (q.shareDevice)
        {
            static const int reserve = []{ const char* v = std::getenv("AIXB200_GEMM_RESERVE_SMS"); return v ? std::atoi(v) : 0; }();
            const uint32_t reservedClusters = static_cast<uint32_t>(std::max(0, reserve)) / 2;
            usable = usable > reservedClusters + 8 ? usable - reservedClusters : usable;
        }
        uint32_t clusters = std::min<uint32_t>(tiles, usable);
        // Remainder tiles are cut along K and shared by all clusters (see WorkIterator) when that saves at least a few
        // stages of idle time per cluster; split-f32 problems keep whole tiles (their partial sums already go through C).
        // Off unless AIXB200_GEMM_SPLITK=1: measured on B200 it helps A^T.B at 4096^3 (+8 %) but costs A.B^T 6 % there
        // and is neutral at 8192^3 - the finisher's epilogue (partials fetched strip by strip) holds its accumulator
        // too long when K is short.
        static const bool splitEnabled = []{ const char* v = std::getenv("AIXB200_GEMM_SPLITK"); return v && v[0] == '1'; }();
        const uint32_t remainder = tiles % static_cast<uint32_t>(maxClusters);
        if (splitEnabled && !tf32 && !q.shareDevice && remainder != 0 && p.kBlocks >= 8)
        {
            const uint64_t units = static_cast<uint64_t>(remainder) * p.kBlocks;
            const uint64_t idleStages = (static_cast<uint64_t>(maxClusters) - remainder) * p.kBlocks / maxClusters;
            if (idleStages >= 6 && units >= static_cast<uint64_t>(maxClusters) && units < 0x7FFFFFFFull)
            {
                clusters = static_cast<uint32_t>(maxClusters);
                p.splitTiles = remainder;
                p.splitUnits = static_cast<uint32_t>(units);
                p.splitWorkspace = static_cast<float*>(device.temporary(static_cast<size_t>(clusters) * 2 * 128 * 256 * sizeof(float)));
                p.splitCounters = reinterpret_cast<uint32_t*>(static_cast<char*>(ctx.scratch) + ctx.scratchBytes);
                if (2ull * remainder * sizeof(uint32_t) > kernels::kGemmCounterBytes) return false;
            }
        }
        // C through shared memory and TMA whenever its rows are 16-byte aligned (AIXB200_GEMM_TMA_STORE=0: direct stores)
        static const bool tmaStoreEnabled = []{ const char* v = std::getenv("AIXB200_GEMM_TMA_STORE"); return !(v && v[0] == '0'); }();
        CUtensorMap mapC = mapA;
        if (tmaStoreEnabled && p.vectorStores)
        {
            const CUtensorMapDataType ctype = q.dtype == F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : (q.dtype == BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
            const size_t es = dtypeSize(q.dtype);
            p.tmaEpilogue = makeMap(&mapC, ctype, q.c, q.n, q.m, q.n * es, static_cast<uint32_t>(128 / es), 32) ? 1u : 0u;
        }
        // Tiles are dealt out at run time while a collective is in flight on this device (its kernel may hold SMs when this
        // one starts: see WorkIterator); alone on the GPU the static deal is 1-3 % faster (measured: 86.2 against 89.3 us at
        // 4096 x 4096 x 1024 f32). AIXB200_GEMM_DYNAMIC=1 / 0: always / never.
        static const int dynamicDeal = []{ const char* v = std::getenv("AIXB200_GEMM_DYNAMIC"); return v ? (v[0] == '0' ? 0 : 1) : -1; }();
        if ((dynamicDeal > 0 || (dynamicDeal < 0 && q.shareDevice)) && ctx.gemmLaunches && p.splitTiles == 0 && tiles < kNoTile &&
            kernels::kGemmRingOffset + static_cast<size_t>(clusters) * kernels::kGemmRingSlots * 8 <= kernels::kGemmCounterBytes)
        {
            char* area = static_cast<char*>(ctx.scratch) + ctx.scratchBytes;
            p.tileCounters = reinterpret_cast<uint32_t*>(area + kernels::kGemmSchedulerOffset);
            p.tileRing = reinterpret_cast<uint64_t*>(area + kernels::kGemmRingOffset);
            // the launch number belongs to the scratch block: counter e % 8 was zeroed by launch e - 4 on the same block
            *ctx.gemmLaunches = (*ctx.gemmLaunches + 1) & 0xFFFFFFu;
            p.tileEpoch = *ctx.gemmLaunches;
        }
        CUtensorMap mapC1 = mapC, mapC2 = mapC;
        p.outputs = 1;
        if (q.bias)
        {
            // folded consumers: every output is a dense m x n f32 tensor that leaves through its own tensor map
            if (!p.halfTerms || !p.tmaEpilogue) return false;
            p.outputs = (q.storeC ? 1u : 0u) | (q.biasOut ? 2u : 0u) | (q.tanhOut ? 4u : 0u);
            p.bias = q.bias;
            p.maxSlot = q.maxSlot;
            if (q.biasOut && !makeMap(&mapC1, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, q.biasOut, q.n, q.m, q.n * 4, 32, 32)) return false;
            if (q.tanhOut && !makeMap(&mapC2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, q.tanhOut, q.n, q.m, q.n * 4, 32, 32)) return false;
            if (q.maxSlot && cudaMemsetAsync(q.maxSlot, 0, 4, ctx.stream) != cudaSuccess) return false;
        }
        if (!tf32)            gemmPairKernel<0><<<2 * clusters, kThreads, pairSmem, ctx.stream>>>(mapA, mapB, mapA16, mapB16, mapC, mapC1, mapC2, p);
        else if (p.halfTerms && q.tanhOut) gemmPairKernel<4><<<2 * clusters, kThreadsHalfTerms, pairSmem, ctx.stream>>>(mapA, mapB, mapA16, mapB16, mapC, mapC1, mapC2, p);
        else if (p.halfTerms && q.bias) gemmPairKernel<3><<<2 * clusters, kThreadsHalfTerms, pairSmem, ctx.stream>>>(mapA, mapB, mapA16, mapB16, mapC, mapC1, mapC2, p);
        else if (p.halfTerms) gemmPairKernel<2><<<2 * clusters, kThreadsHalfTerms, pairSmem, ctx.stream>>>(mapA, mapB, mapA16, mapB16, mapC, mapC1, mapC2, p);
        else                  gemmPairKernel<1><<<2 * clusters, kThreads, pairSmem, ctx.stream>>>(mapA, mapB, mapA16, mapB16, mapC, mapC1, mapC2, p);
        if (ctx.launches) ++*ctx.launches;
        return true;
    }
    if (q.bias) return false;
    const uint32_t grid = std::min<uint32_t>(tiles, static_cast<uint32_t>(ctx.smCount));
    if (tf32) gemmKernel<true><<<grid, kThreads, smemBytes, ctx.stream>>>(mapA, mapB, mapA16, mapB16, p);
    else      gemmKernel<false><<<grid, kThreads, smemBytes, ctx.stream>>>(mapA, mapB, mapA16, mapB16, p);
    if (ctx.launches) ++*ctx.launches;
    return true;
}

}   // namespace aixb200::gemm
