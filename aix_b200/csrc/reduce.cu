// Reduction kernels: warp-shuffle + shared-memory trees.
//
// Replaces the reference's staged tree reductions (aixDeviceMetalShaders.hpp:1539-1664 for sum/max and :1824-2160
// for reduceTo/maxTo; host orchestration aixDeviceMetal.cpp:296-445, 773-983, 2066-2192). The reference makes
// log_1024(n) passes over a full-size temporary; here a full reduction is ONE launch: every CTA streams its share
// with 128-bit loads, leaves one 64-bit partial in scratch, and the CTA that takes the last ticket folds the
// partials in a fixed order (so results are reproducible run to run).
//
// Accumulation: floating sums are kept in float per thread (a few hundred terms at most) and in double across
// threads and CTAs; f16/bf16 therefore accumulate in at least f32 and round once at the end. Integer sums wrap in
// the storage type exactly like the sequential loop of the reference (aixDeviceCPU.cpp:140-152), max is exact.
#include "dtypes.cuh"
#include "kernels.hpp"

#include <algorithm>
#include <atomic>

namespace aixb200::kernels
{

using namespace aixb200::dev;

namespace
{

constexpr int kBlock = 256;

struct StridedSrc
{
    int      rank;
    uint64_t shape[MAX_RANK];
    uint64_t strides[MAX_RANK];
};

__device__ __forceinline__ uint64_t stridedOffset(uint64_t i, const StridedSrc& s)
{
    uint64_t off = 0;
    for (int d = s.rank - 1; d >= 1; --d)
    {
        const uint64_t q = i / s.shape[d];
        off += (i - q * s.shape[d]) * s.strides[d];
        i = q;
    }
    return s.rank > 0 ? off + i * s.strides[0] : off;
}

// ------------------------------------------------------------------------------------------------------------
// Full reduction, one launch. partials: gridDim.x 64-bit slots; ticket: one uint32 that is zero on entry and
// left at zero on exit.
// ------------------------------------------------------------------------------------------------------------
template <int DT, bool IsMax, bool Dense>
__global__ void __launch_bounds__(kBlock) reduceAllKernel(const typename Elem<DT>::S* __restrict__ src, uint64_t n, StridedSrc layout,
                                                          unsigned long long* partials, unsigned int* ticket,
                                                          typename Elem<DT>::S* dst)
{
    typedef Reduce<DT, IsMax> R;
    typedef typename R::S S;
    typedef typename R::A A;
    typedef typename R::W W;
    constexpr int VEC = 16 / sizeof(S);
    __shared__ W smem[32];
    __shared__ bool isLast;

    A acc[VEC];
    #pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = R::init();

    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x;
    const uint64_t threads = static_cast<uint64_t>(gridDim.x) * kBlock;
    if (Dense)
    {
        // src is 16-byte aligned (checked by the launcher)
        const uint64_t nvec = n / VEC;
        const Pack<S, VEC>* vsrc = reinterpret_cast<const Pack<S, VEC>*>(src);
        uint64_t i = tid;
        for (; i + 3 * threads < nvec; i += 4 * threads)      // four packs (64 bytes) in flight per thread
        {
            const Pack<S, VEC> p0 = vsrc[i], p1 = vsrc[i + threads], p2 = vsrc[i + 2 * threads], p3 = vsrc[i + 3 * threads];
            #pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = R::step(R::step(R::step(R::step(acc[e], p0.v[e]), p1.v[e]), p2.v[e]), p3.v[e]);
        }
        for (; i < nvec; i += threads)
        {
            const Pack<S, VEC> p0 = vsrc[i];
            #pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = R::step(acc[e], p0.v[e]);
        }
        const uint64_t t = nvec * VEC + tid;
        if (t < n) acc[0] = R::step(acc[0], src[t]);
    }
    else
    {
        for (uint64_t i = tid; i < n; i += threads) acc[0] = R::step(acc[0], src[stridedOffset(i, layout)]);
    }

    W w = R::widen(acc[0]);
    #pragma unroll
    for (int e = 1; e < VEC; ++e) w = R::merge(w, R::widen(acc[e]));
    w = blockReduce<R>(w, smem);

    if (threadIdx.x == 0)
    {
        partials[blockIdx.x] = *reinterpret_cast<unsigned long long*>(&w);
        __threadfence();
        const unsigned int t = atomicAdd(ticket, 1u);
        isLast = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!isLast) return;
    __threadfence();
    W total = R::identityW();
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += kBlock)
    {
        unsigned long long bits = __ldcg(&partials[b]);
        total = R::merge(total, *reinterpret_cast<W*>(&bits));
    }
    total = blockReduce<R>(total, smem);
    if (threadIdx.x == 0)
    {
        dst[0] = R::finish(total);
        *ticket = 0;
    }
}

template <int DT>
void launchReduceAll(const LaunchContext& ctx, bool isMax, const View& src, void* dst, void* scratch, size_t scratchBytes)
{
    typedef typename Elem<DT>::S S;
    auto ticket = static_cast<unsigned int*>(scratch);
    auto partials = reinterpret_cast<unsigned long long*>(static_cast<char*>(scratch) + kScratchCounterBytes);
    const size_t maxBlocks = std::min<size_t>(kMaxReduceBlocks, (scratchBytes - kScratchCounterBytes) / 8);
    const S* base = reinterpret_cast<const S*>(src.firstByte());
    const bool dense = src.isDense() && (reinterpret_cast<uintptr_t>(base) % 16 == 0);
    StridedSrc layout{};
    layout.rank = src.rank;
    for (int d = 0; d < src.rank; ++d) { layout.shape[d] = src.shape[d]; layout.strides[d] = src.strides[d]; }
    const uint64_t perBlock = static_cast<uint64_t>(kBlock) * (dense ? 4 * (16 / sizeof(S)) : 1);
    uint64_t blocks = (src.size + perBlock - 1) / perBlock;
    // A grid-stride kernel: no more CTAs than are resident at once (what the kernel's registers allow, at most 8 per SM) -
    // a partial second wave would run at a fraction of the bandwidth while everything else has finished.
    auto residentPerSm = [](const void* kernel)
    {
        int perSm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, kBlock, 0) != cudaSuccess || perSm <= 0) { cudaGetLastError(); perSm = 8; }
        return std::min(perSm, 8);
    };
    static const int resident[4] = {residentPerSm(reinterpret_cast<const void*>(&reduceAllKernel<DT, false, false>)),
                                    residentPerSm(reinterpret_cast<const void*>(&reduceAllKernel<DT, false, true>)),
                                    residentPerSm(reinterpret_cast<const void*>(&reduceAllKernel<DT, true, false>)),
                                    residentPerSm(reinterpret_cast<const void*>(&reduceAllKernel<DT, true, true>))};
    const int perSm = resident[(isMax ? 2 : 0) + (dense ? 1 : 0)];
    blocks = std::max<uint64_t>(1, std::min<uint64_t>(blocks, std::min<uint64_t>(maxBlocks, static_cast<uint64_t>(ctx.smCount) * perSm)));
    auto out = static_cast<S*>(dst);
    const unsigned int grid = static_cast<unsigned int>(blocks);
    if (isMax)
    {
        if (dense) reduceAllKernel<DT, true, true><<<grid, kBlock, 0, ctx.stream>>>(base, src.size, layout, partials, ticket, out);
        else       reduceAllKernel<DT, true, false><<<grid, kBlock, 0, ctx.stream>>>(base, src.size, layout, partials, ticket, out);
    }
    else
    {
        if (dense) reduceAllKernel<DT, false, true><<<grid, kBlock, 0, ctx.stream>>>(base, src.size, layout, partials, ticket, out);
        else       reduceAllKernel<DT, false, false><<<grid, kBlock, 0, ctx.stream>>>(base, src.size, layout, partials, ticket, out);
    }
    if (ctx.launches) ++*ctx.launches;
}

// ------------------------------------------------------------------------------------------------------------
// dst[k] (+)= fold over r of src[k * keptStride + r]: one CTA (long rows) or one warp (short rows) per output.
// ------------------------------------------------------------------------------------------------------------
template <int DT, bool IsMax, bool WarpPerRow>
__global__ void __launch_bounds__(kBlock, 8) reduceRowsKernel(const typename Elem<DT>::S* __restrict__ src, uint64_t rows, uint64_t cols,
                                                           uint64_t rowStride, typename Elem<DT>::S* dst)
{
    typedef Reduce<DT, IsMax> R;
    typedef typename R::S S;
    typedef typename R::A A;
    typedef typename R::W W;
    constexpr int VEC = 16 / sizeof(S);
    __shared__ W smem[32];
    const int lanes = WarpPerRow ? 32 : kBlock;
    const int lane = WarpPerRow ? (threadIdx.x & 31) : threadIdx.x;
    const uint64_t rowsPerBlock = WarpPerRow ? kBlock / 32 : 1;
    for (uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * rowsPerBlock; row0 < rows; row0 += static_cast<uint64_t>(gridDim.x) * rowsPerBlock)
    {
        const uint64_t row = row0 + (WarpPerRow ? (threadIdx.x >> 5) : 0);
        W w = R::identityW();
        if (row < rows)
        {
            const S* p = src + row * rowStride;
            A acc[VEC];
            #pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = R::init();
            // scalar head up to the first 16-byte boundary, packs in the middle, scalar tail
            const uintptr_t addr = reinterpret_cast<uintptr_t>(p);
            uint64_t head = ((16 - (addr & 15)) & 15) / sizeof(S);
            if (head > cols) head = cols;
            if (static_cast<uint64_t>(lane) < head) acc[0] = R::step(acc[0], p[lane]);
            const uint64_t nvec = (cols - head) / VEC;
            const Pack<S, VEC>* vp = reinterpret_cast<const Pack<S, VEC>*>(p + head);
            uint64_t i = lane;
            for (; i + 3 * lanes < nvec; i += 4 * lanes)         // four independent 128-bit loads per thread
            {
                const Pack<S, VEC> p0 = vp[i], p1 = vp[i + lanes], p2 = vp[i + 2 * lanes], p3 = vp[i + 3 * lanes];
                #pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] = R::step(R::step(R::step(R::step(acc[e], p0.v[e]), p1.v[e]), p2.v[e]), p3.v[e]);
            }
            for (; i < nvec; i += lanes)
            {
                const Pack<S, VEC> pk = vp[i];
                #pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] = R::step(acc[e], pk.v[e]);
            }
            const uint64_t t = head + nvec * VEC + lane;
            if (t < cols) acc[0] = R::step(acc[0], p[t]);
            w = R::widen(acc[0]);
            #pragma unroll
            for (int e = 1; e < VEC; ++e) w = R::merge(w, R::widen(acc[e]));
        }
        if (WarpPerRow)
        {
            #pragma unroll
            for (int d = 16; d > 0; d >>= 1) w = R::merge(w, shuffleDown<W>(w, d));
            if (lane == 0 && row < rows) dst[row] = R::finish(R::merge(R::liftStored(dst[row]), w));
        }
        else
        {
            w = blockReduce<R>(w, smem);
            if (threadIdx.x == 0) dst[row] = R::finish(R::merge(R::liftStored(dst[row]), w));
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// dst[k] (+)= fold over r of src[r * rowStride + k] (column sums). Each thread owns one column of a 32-column
// tile, the 8 warps of a CTA take interleaved rows of the CTA's row slab; slabs are combined through scratch so the
// result does not depend on scheduling.
// ------------------------------------------------------------------------------------------------------------
template <int DT, bool IsMax>
__global__ void __launch_bounds__(kBlock) reduceColsKernel(const typename Elem<DT>::S* __restrict__ src, uint64_t rows, uint64_t cols,
                                                           uint64_t rowStride, uint64_t rowsPerSlab, unsigned long long* partials,
                                                           typename Elem<DT>::S* dst)
{
    typedef Reduce<DT, IsMax> R;
    typedef typename R::S S;
    typedef typename R::A A;
    typedef typename R::W W;
    constexpr int kWarps = kBlock / 32;
    __shared__ W tile[kWarps][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t col = static_cast<uint64_t>(blockIdx.x) * 32 + lane;
    const uint64_t rowBegin = static_cast<uint64_t>(blockIdx.y) * rowsPerSlab;
    const uint64_t rowEnd = min(rows, rowBegin + rowsPerSlab);
    A acc0 = R::init(), acc1 = R::init();
    if (col < cols)
    {
        uint64_t r = rowBegin + warp;
        for (; r + kWarps < rowEnd; r += 2 * kWarps)
        {
            const S a = src[r * rowStride + col], b = src[(r + kWarps) * rowStride + col];
            acc0 = R::step(acc0, a);
            acc1 = R::step(acc1, b);
        }
        if (r < rowEnd) acc0 = R::step(acc0, src[r * rowStride + col]);
    }
    tile[warp][lane] = R::merge(R::widen(acc0), R::widen(acc1));
    __syncthreads();
    if (warp == 0 && col < cols)
    {
        W w = tile[0][lane];
        #pragma unroll
        for (int k = 1; k < kWarps; ++k) w = R::merge(w, tile[k][lane]);
        if (gridDim.y == 1) dst[col] = R::finish(R::merge(R::liftStored(dst[col]), w));
        else partials[static_cast<uint64_t>(blockIdx.y) * cols + col] = *reinterpret_cast<unsigned long long*>(&w);
    }
}

// Same reduction when rows are 16-byte aligned and the column count is a multiple of the pack width: every lane owns
// one pack of adjacent columns, so a warp reads 512 contiguous bytes of a row per instruction.
template <int DT, bool IsMax>
__global__ void __launch_bounds__(kBlock) reduceColsVecKernel(const typename Elem<DT>::S* __restrict__ src, uint64_t rows, uint64_t cols,
                                                              uint64_t rowStride, uint64_t rowsPerSlab, unsigned long long* partials,
                                                              typename Elem<DT>::S* dst)
{
    typedef Reduce<DT, IsMax> R;
    typedef typename R::S S;
    typedef typename R::A A;
    typedef typename R::W W;
    constexpr int VEC = 16 / sizeof(S);
    constexpr int kWarps = kBlock / 32;
    __shared__ W tile[kWarps][32 * VEC + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t col0 = (static_cast<uint64_t>(blockIdx.x) * 32 + lane) * VEC;
    const uint64_t rowBegin = static_cast<uint64_t>(blockIdx.y) * rowsPerSlab;
    const uint64_t rowEnd = min(rows, rowBegin + rowsPerSlab);
    A acc0[VEC], acc1[VEC];
    #pragma unroll
    for (int e = 0; e < VEC; ++e) { acc0[e] = R::init(); acc1[e] = R::init(); }
    if (col0 < cols)
    {
        uint64_t r = rowBegin + warp;
        for (; r + kWarps < rowEnd; r += 2 * kWarps)
        {
            const Pack<S, VEC> a = *reinterpret_cast<const Pack<S, VEC>*>(src + r * rowStride + col0);
            const Pack<S, VEC> b = *reinterpret_cast<const Pack<S, VEC>*>(src + (r + kWarps) * rowStride + col0);
            #pragma unroll
            for (int e = 0; e < VEC; ++e) { acc0[e] = R::step(acc0[e], a.v[e]); acc1[e] = R::step(acc1[e], b.v[e]); }
        }
        if (r < rowEnd)
        {
            const Pack<S, VEC> a = *reinterpret_cast<const Pack<S, VEC>*>(src + r * rowStride + col0);
            #pragma unroll
            for (int e = 0; e < VEC; ++e) acc0[e] = R::step(acc0[e], a.v[e]);
        }
    }
    #pragma unroll
    for (int e = 0; e < VEC; ++e) tile[warp][lane * VEC + e] = R::merge(R::widen(acc0[e]), R::widen(acc1[e]));
    __syncthreads();
    // 32 * VEC columns per CTA, folded over the warps by the first threads
    for (int c = threadIdx.x; c < 32 * VEC; c += kBlock)
    {
        const uint64_t col = static_cast<uint64_t>(blockIdx.x) * 32 * VEC + c;
        if (col >= cols) continue;
        W w = tile[0][c];
        #pragma unroll
        for (int k = 1; k < kWarps; ++k) w = R::merge(w, tile[k][c]);
        if (gridDim.y == 1) dst[col] = R::finish(R::merge(R::liftStored(dst[col]), w));
        else partials[static_cast<uint64_t>(blockIdx.y) * cols + col] = *reinterpret_cast<unsigned long long*>(&w);
    }
}

template <int DT, bool IsMax>
__global__ void __launch_bounds__(kBlock) combineSlabsKernel(const unsigned long long* partials, uint64_t cols, unsigned int slabs,
                                                             typename Elem<DT>::S* dst)
{
    typedef Reduce<DT, IsMax> R;
    typedef typename R::W W;
    const uint64_t col = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x;
    if (col >= cols) return;
    W w = R::liftStored(dst[col]);
    for (unsigned int s = 0; s < slabs; ++s)
    {
        unsigned long long bits = partials[static_cast<uint64_t>(s) * cols + col];
        w = R::merge(w, *reinterpret_cast<W*>(&bits));
    }
    dst[col] = R::finish(w);
}

// ------------------------------------------------------------------------------------------------------------
// Any other pattern: one thread per output element walks the reduced coordinates.
// ------------------------------------------------------------------------------------------------------------
struct GenericDims
{
    int      keptRank, reducedRank;
    uint64_t keptExtent[MAX_RANK], keptStride[MAX_RANK];
    uint64_t redExtent[MAX_RANK], redStride[MAX_RANK];
    uint64_t outputs, reducedCount;
};

template <int DT, bool IsMax>
__global__ void __launch_bounds__(kBlock) reduceGenericKernel(const typename Elem<DT>::S* __restrict__ src, GenericDims g,
                                                              typename Elem<DT>::S* dst)
{
    typedef Reduce<DT, IsMax> R;
    typedef typename R::W W;
    const uint64_t o = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x;
    if (o >= g.outputs) return;
    uint64_t base = 0, rem = o;
    for (int d = g.keptRank - 1; d >= 0; --d)
    {
        const uint64_t q = rem / g.keptExtent[d];
        base += (rem - q * g.keptExtent[d]) * g.keptStride[d];
        rem = q;
    }
    W w = R::liftStored(dst[o]);
    for (uint64_t r = 0; r < g.reducedCount; ++r)
    {
        uint64_t off = base, rr = r;
        for (int d = g.reducedRank - 1; d >= 0; --d)
        {
            const uint64_t q = rr / g.redExtent[d];
            off += (rr - q * g.redExtent[d]) * g.redStride[d];
            rr = q;
        }
        w = R::merge(w, R::liftStored(src[off]));
    }
    dst[o] = R::finish(w);
}

template <int DT>
void launchReduceInto(const LaunchContext& ctx, bool isMax, const void* srcRaw, const ReduceDim* dims, int rank, void* dstRaw)
{
    typedef typename Elem<DT>::S S;
    auto src = static_cast<const S*>(srcRaw);
    auto dst = static_cast<S*>(dstRaw);
    auto count = [&](int* bump) { if (ctx.launches) *ctx.launches += *bump; };
    int one = 1, two = 2;

    // [kept][reduced, contiguous]  -> row reduction
    if (rank == 2 && dims[0].kept && !dims[1].kept && dims[1].stride == 1)
    {
        const uint64_t rows = dims[0].extent, cols = dims[1].extent;
        // A warp per row needs no block-wide synchronisation; it wins whenever there are enough rows to fill the GPU
        // with warps and a row is short enough (<= 64 KiB) for one warp to stream.
        const bool warpPerRow = cols < 1024 || (cols * sizeof(S) <= 65536 && rows >= static_cast<uint64_t>(ctx.smCount) * 16);
        const uint64_t blocksWanted = warpPerRow ? (rows + 7) / 8 : rows;
        const unsigned int grid = static_cast<unsigned int>(std::max<uint64_t>(1, std::min<uint64_t>(blocksWanted, static_cast<uint64_t>(ctx.smCount) * 16)));
        if (isMax)
        {
            if (warpPerRow) reduceRowsKernel<DT, true, true><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, dst);
            else            reduceRowsKernel<DT, true, false><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, dst);
        }
        else
        {
            if (warpPerRow) reduceRowsKernel<DT, false, true><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, dst);
            else            reduceRowsKernel<DT, false, false><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, dst);
        }
        count(&one);
        return;
    }
    // [reduced][kept, contiguous]  -> column reduction
    if (rank == 2 && !dims[0].kept && dims[1].kept && dims[1].stride == 1)
    {
        const uint64_t rows = dims[0].extent, cols = dims[1].extent;
        constexpr uint64_t kVec = 16 / sizeof(S);
        const bool vectorised = cols % kVec == 0 && (dims[0].stride * sizeof(S)) % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0;
        const uint64_t colTiles = vectorised ? (cols + 32 * kVec - 1) / (32 * kVec) : (cols + 31) / 32;
        auto partials = reinterpret_cast<unsigned long long*>(static_cast<char*>(ctx.scratch) + kScratchCounterBytes);
        const uint64_t partialCapacity = (ctx.scratchBytes - kScratchCounterBytes) / 8;
        uint64_t slabs = std::max<uint64_t>(1, (static_cast<uint64_t>(ctx.smCount) * 4 + colTiles - 1) / colTiles);
        slabs = std::min<uint64_t>(slabs, std::max<uint64_t>(1, rows / 32));
        slabs = std::min<uint64_t>(slabs, std::max<uint64_t>(1, partialCapacity / std::max<uint64_t>(cols, 1)));
        slabs = std::min<uint64_t>(slabs, 65535);
        const uint64_t rowsPerSlab = (rows + slabs - 1) / slabs;
        slabs = (rows + rowsPerSlab - 1) / rowsPerSlab;
        dim3 grid(static_cast<unsigned int>(colTiles), static_cast<unsigned int>(slabs));
        if (vectorised)
        {
            if (isMax) reduceColsVecKernel<DT, true><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, rowsPerSlab, partials, dst);
            else       reduceColsVecKernel<DT, false><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, rowsPerSlab, partials, dst);
        }
        else if (isMax) reduceColsKernel<DT, true><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, rowsPerSlab, partials, dst);
        else            reduceColsKernel<DT, false><<<grid, kBlock, 0, ctx.stream>>>(src, rows, cols, dims[0].stride, rowsPerSlab, partials, dst);
        if (slabs > 1)
        {
            const unsigned int cgrid = static_cast<unsigned int>((cols + kBlock - 1) / kBlock);
            if (isMax) combineSlabsKernel<DT, true><<<cgrid, kBlock, 0, ctx.stream>>>(partials, cols, static_cast<unsigned int>(slabs), dst);
            else       combineSlabsKernel<DT, false><<<cgrid, kBlock, 0, ctx.stream>>>(partials, cols, static_cast<unsigned int>(slabs), dst);
            count(&two);
        }
        else count(&one);
        return;
    }
    GenericDims g{};
    g.outputs = 1;
    g.reducedCount = 1;
    for (int d = 0; d < rank; ++d)
    {
        if (dims[d].kept) { g.keptExtent[g.keptRank] = dims[d].extent; g.keptStride[g.keptRank] = dims[d].stride; ++g.keptRank; g.outputs *= dims[d].extent; }
        else { g.redExtent[g.reducedRank] = dims[d].extent; g.redStride[g.reducedRank] = dims[d].stride; ++g.reducedRank; g.reducedCount *= dims[d].extent; }
    }
    const unsigned int grid = static_cast<unsigned int>((g.outputs + kBlock - 1) / kBlock);
    if (isMax) reduceGenericKernel<DT, true><<<grid, kBlock, 0, ctx.stream>>>(src, g, dst);
    else       reduceGenericKernel<DT, false><<<grid, kBlock, 0, ctx.stream>>>(src, g, dst);
    count(&one);
}

}   // namespace

// ------------------------------------------------------------------------------------------------------------
// Scratch that is part of the library image instead of the heap: one ticket word (first 256 bytes) and 4064 partial
// slots. Every GPU that loads the library carries these 32 KiB until the process exits. In host code the array's
// name is only a stand-in; the device address comes from cudaGetSymbolAddress, once per device.
// ------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_staticReduceScratch[kStaticScratchBytes];

const char* sumWithStaticScratch(const LaunchContext& ctx, int ordinal, const View& src, void* dst)
{
    constexpr int kMaxDevices = 64;
    static std::atomic<void*> addresses[kMaxDevices] = {};      // two handles may make their first call from two threads
    if (ordinal < 0 || ordinal >= kMaxDevices) return "device ordinal out of range for the static scratch table";
    void* scratch = addresses[ordinal].load(std::memory_order_acquire);
    if (!scratch)
    {
        // First call on this device (the device is current): resolve the array's device address.
        cudaError_t e = cudaGetSymbolAddress(&scratch, g_staticReduceScratch);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        addresses[ordinal].store(scratch, std::memory_order_release);
    }
    // The ticket must start at zero; a launch that was cut short could have left it raised.
    cudaError_t e = cudaMemsetAsync(scratch, 0, kScratchCounterBytes, ctx.stream);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    reduceAllWithScratch(ctx, false, src, dst, scratch, kStaticScratchBytes);
    e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

void reduceAllWithScratch(const LaunchContext& ctx, bool isMax, const View& src, void* dst, void* scratch, size_t scratchBytes)
{
    AIXB200_DISPATCH_DTYPE(src.dtype, launchReduceAll, ctx, isMax, src, dst, scratch, scratchBytes);
}

void reduceAll(const LaunchContext& ctx, bool isMax, const View& src, void* dst)
{
    reduceAllWithScratch(ctx, isMax, src, dst, ctx.scratch, ctx.scratchBytes);
}

void reduceInto(const LaunchContext& ctx, bool isMax, uint32_t dtype, const void* src, const ReduceDim* dims, int rank, void* dst)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchReduceInto, ctx, isMax, src, dims, rank, dst);
}

}   // namespace aixb200::kernels
