// Fixed kernels off the hot path: argmax family, CUDA-core matmul for shapes and types the tensor-core GEMM does
// not take, and the data-movement ops of the device interface (transpose, sliceSet, tril/triu, indexSelect,
// indexAdd). Index arithmetic follows the reference's CPU loops (aixDeviceCPU.cpp:258-622) so results are
// identical; each kernel is the obvious one-thread-per-element form of the corresponding loop.
#include "dtypes.cuh"
#include "kernels.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace aixb200::kernels
{

using namespace aixb200::dev;

namespace
{

constexpr int kBlock = 256;

__device__ __forceinline__ uint64_t layoutOffset(uint64_t i, const Layout& l)
{
    uint64_t off = 0;
    for (int d = l.rank - 1; d >= 0; --d)
    {
        const uint64_t q = i / l.shape[d];
        off += (i - q * l.shape[d]) * l.strides[d];
        i = q;
    }
    return off;
}

inline uint32_t* badIndexWord(const LaunchContext& ctx) { return reinterpret_cast<uint32_t*>(static_cast<char*>(ctx.scratch) + kScratchBadIndexOffset); }

inline unsigned int gridFor(uint64_t count, int smCount)
{
    const uint64_t blocks = (count + kBlock - 1) / kBlock;
    return static_cast<unsigned int>(std::max<uint64_t>(1, std::min<uint64_t>(blocks, static_cast<uint64_t>(smCount) * 16)));
}

// ---- argmax over everything: first maximal index wins (aixDeviceCPU.cpp:258-272) ----------------------------------
// Stage 1: every CTA scans a grid-strided share (each thread sees its indices in increasing order and keeps the first
// strictly greater value), folds it with the tie rule "equal value -> smaller index" and leaves one (value, index)
// partial in scratch; the CTA that draws the last ticket folds the partials with the same rule, so the result is the
// one the reference's sequential loop finds, whatever the grid. The one-hot form needs the winner in every CTA and
// takes a second launch. (The reference runs a multi-pass tree, aixDeviceMetalShaders.hpp:1667-1800.)
constexpr int kArgmaxBlock = 256;
constexpr size_t kArgmaxTicketOffset = 64, kArgmaxWinnerOffset = 72;
constexpr unsigned kArgmaxMaxBlocks = 1024;

template <class V> __device__ __forceinline__ void argmaxFold(V& bestV, uint64_t& bestI, V otherV, uint64_t otherI)
{
    if (otherI != ~0ull && (bestI == ~0ull || otherV > bestV || (otherV == bestV && otherI < bestI))) { bestV = otherV; bestI = otherI; }
}

template <int DT>
__global__ void __launch_bounds__(kArgmaxBlock) argmaxAllKernel(const typename Elem<DT>::S* __restrict__ src, Layout layout, uint64_t n,
                                                                typename Elem<DT>::V* partialV, uint64_t* partialI, unsigned int* ticket,
                                                                uint64_t* winnerSlot, int32_t* dst, bool oneHot)
{
    typedef Elem<DT> E;
    typedef typename E::V V;
    __shared__ V sharedV[kArgmaxBlock];
    __shared__ uint64_t sharedI[kArgmaxBlock];
    __shared__ bool isLast;
    V best = E::lowest();
    uint64_t bestIdx = ~0ull;
    const bool dense = layout.rank <= 1 && (layout.rank == 0 || layout.strides[0] == 1);
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kArgmaxBlock + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * kArgmaxBlock)
    {
        const V v = E::load(src[dense ? i : layoutOffset(i, layout)]);
        if (bestIdx == ~0ull || v > best) { best = v; bestIdx = i; }
    }
    auto blockFold = [&]()
    {
        sharedV[threadIdx.x] = best;
        sharedI[threadIdx.x] = bestIdx;
        __syncthreads();
        for (int s = kArgmaxBlock / 2; s > 0; s >>= 1)
        {
            if (threadIdx.x < s)
            {
                V v = sharedV[threadIdx.x];
                uint64_t i = sharedI[threadIdx.x];
                argmaxFold(v, i, sharedV[threadIdx.x + s], sharedI[threadIdx.x + s]);
                sharedV[threadIdx.x] = v;
                sharedI[threadIdx.x] = i;
            }
            __syncthreads();
        }
    };
    blockFold();
    if (threadIdx.x == 0)
    {
        partialV[blockIdx.x] = sharedV[0];
        partialI[blockIdx.x] = sharedI[0];
        __threadfence();
        isLast = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!isLast) return;
    __threadfence();
    best = E::lowest();
    bestIdx = ~0ull;
    for (unsigned b = threadIdx.x; b < gridDim.x; b += kArgmaxBlock)
        argmaxFold(best, bestIdx, *const_cast<volatile V*>(partialV + b), *const_cast<volatile uint64_t*>(partialI + b));
    blockFold();
    if (threadIdx.x == 0)
    {
        // The sequential loop of the reference keeps index 0 unless a strictly greater value appears.
        const uint64_t winner = sharedI[0] == ~0ull ? 0 : sharedI[0];
        if (oneHot) *winnerSlot = winner; else dst[0] = static_cast<int32_t>(winner);
        *ticket = 0;
    }
}

__global__ void __launch_bounds__(kBlock) oneHotKernel(int32_t* dst, uint64_t n, const uint64_t* winnerSlot)
{
    const uint64_t winner = *winnerSlot;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * kBlock)
        dst[i] = (i == winner) ? 1 : 0;
}

template <int DT>
void launchArgmaxAll(const LaunchContext& ctx, const View& src, int32_t* dst, bool oneHot, uint64_t count)
{
    typedef typename Elem<DT>::V V;
    Layout l{};
    l.rank = src.rank;
    for (int d = 0; d < src.rank; ++d) { l.shape[d] = src.shape[d]; l.strides[d] = src.strides[d]; }
    char* scratch = static_cast<char*>(ctx.scratch);
    auto partialV = reinterpret_cast<V*>(scratch + kScratchCounterBytes);
    auto partialI = reinterpret_cast<uint64_t*>(scratch + kScratchCounterBytes + kArgmaxMaxBlocks * 8);
    auto ticket = reinterpret_cast<unsigned int*>(scratch + kArgmaxTicketOffset);
    auto winner = reinterpret_cast<uint64_t*>(scratch + kArgmaxWinnerOffset);
    const uint64_t wanted = (count + kArgmaxBlock * 8 - 1) / (kArgmaxBlock * 8);
    const unsigned grid = static_cast<unsigned>(std::max<uint64_t>(1, std::min<uint64_t>(wanted, std::min<uint64_t>(kArgmaxMaxBlocks, static_cast<uint64_t>(ctx.smCount) * 4))));
    argmaxAllKernel<DT><<<grid, kArgmaxBlock, 0, ctx.stream>>>(reinterpret_cast<const typename Elem<DT>::S*>(src.firstByte()), l, count, partialV, partialI,
                                                               ticket, winner, dst, oneHot);
    if (ctx.launches) ++*ctx.launches;
    if (oneHot)
    {
        oneHotKernel<<<gridFor(count, ctx.smCount), kBlock, 0, ctx.stream>>>(dst, count, winner);
        if (ctx.launches) ++*ctx.launches;
    }
}

// ---- argmax along one dimension: one thread per output (aixDeviceCPU.cpp:275-352) ---------------------------
struct AlongDims
{
    int      rank, reducedDim;
    uint64_t extent[MAX_RANK], stride[MAX_RANK];
    uint64_t outputs;
};

template <int DT>
__global__ void __launch_bounds__(kBlock) argmaxAlongKernel(const typename Elem<DT>::S* __restrict__ src, AlongDims g, int32_t* dst, bool oneHot)
{
    typedef Elem<DT> E;
    typedef typename E::V V;
    const uint64_t o = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x;
    if (o >= g.outputs) return;
    // decompose the output index over all dimensions except the reduced one
    uint64_t rem = o, base = 0, flatOuter = 0, flatInnerStride = 1;
    uint64_t coords[MAX_RANK];
    for (int d = g.rank - 1; d >= 0; --d)
    {
        if (d == g.reducedDim) { coords[d] = 0; continue; }
        const uint64_t q = rem / g.extent[d];
        coords[d] = rem - q * g.extent[d];
        base += coords[d] * g.stride[d];
        rem = q;
    }
    V best = E::load(src[base]);
    uint64_t bestK = 0;
    for (uint64_t k = 1; k < g.extent[g.reducedDim]; ++k)
    {
        const V v = E::load(src[base + k * g.stride[g.reducedDim]]);
        if (v > best) { best = v; bestK = k; }
    }
    if (!oneHot) { dst[o] = static_cast<int32_t>(bestK); return; }
    // flat row-major index of the winner in the source shape
    coords[g.reducedDim] = bestK;
    for (int d = g.rank - 1; d >= 0; --d) { flatOuter += coords[d] * flatInnerStride; flatInnerStride *= g.extent[d]; }
    dst[flatOuter] = 1;
}

template <int DT>
void launchArgmaxAlong(const LaunchContext& ctx, const void* src, const ReduceDim* dims, int rank, int reducedDim, int32_t* dst, bool oneHot)
{
    AlongDims g{};
    g.rank = rank;
    g.reducedDim = reducedDim;
    g.outputs = 1;
    for (int d = 0; d < rank; ++d)
    {
        g.extent[d] = dims[d].extent;
        g.stride[d] = dims[d].stride;
        if (d != reducedDim) g.outputs *= dims[d].extent;
    }
    const unsigned int grid = static_cast<unsigned int>((g.outputs + kBlock - 1) / kBlock);
    argmaxAlongKernel<DT><<<grid, kBlock, 0, ctx.stream>>>(static_cast<const typename Elem<DT>::S*>(src), g, dst, oneHot);
    if (ctx.launches) ++*ctx.launches;
}

// ---- CUDA-core matmul: 64x64 tile, 16-deep k step, 4x4 outputs per thread, any strides -----------------------
// Accumulates in float for f32/f16/bf16, double for f64, and wraps for integers (aixDeviceCPU.cpp:355-388 accumulates
// in the storage type; for 16-bit floats the wider accumulator is deliberate).
template <int DT> struct MatAcc { typedef typename Elem<DT>::SumA T; };

template <int DT>
__global__ void __launch_bounds__(256) matmulSimtKernel(const typename Elem<DT>::S* __restrict__ a, uint64_t ars, uint64_t acs,
                                                        const typename Elem<DT>::S* __restrict__ b, uint64_t brs, uint64_t bcs,
                                                        typename Elem<DT>::S* __restrict__ c, uint64_t m, uint64_t n, uint64_t k)
{
    typedef Elem<DT> E;
    typedef typename MatAcc<DT>::T A;
    __shared__ A as[16][64 + 4];
    __shared__ A bs[16][64 + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint64_t row0 = static_cast<uint64_t>(blockIdx.y) * 64, col0 = static_cast<uint64_t>(blockIdx.x) * 64;
    A acc[4][4];
    #pragma unroll
    for (int i = 0; i < 4; ++i)
        #pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = A(0);
    for (uint64_t k0 = 0; k0 < k; k0 += 16)
    {
        for (int t = threadIdx.x; t < 16 * 64; t += 256)
        {
            const int kk = t & 15, rr = t >> 4;             // A tile: 64 rows x 16 k
            const uint64_t r = row0 + rr, kg = k0 + kk;
            as[kk][rr] = (r < m && kg < k) ? static_cast<A>(E::load(a[r * ars + kg * acs])) : A(0);
            const int cc = t & 63, kb = t >> 6;             // B tile: 16 k x 64 cols
            const uint64_t cg = col0 + cc, kg2 = k0 + kb;
            bs[kb][cc] = (cg < n && kg2 < k) ? static_cast<A>(E::load(b[kg2 * brs + cg * bcs])) : A(0);
        }
        __syncthreads();
        #pragma unroll
        for (int kk = 0; kk < 16; ++kk)
        {
            A av[4], bv[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
            #pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tx * 4 + j];
            #pragma unroll
            for (int i = 0; i < 4; ++i)
                #pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
    #pragma unroll
    for (int i = 0; i < 4; ++i)
        #pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const uint64_t r = row0 + ty * 4 + i, cidx = col0 + tx * 4 + j;
            if (r < m && cidx < n) c[r * n + cidx] = E::fromSum(static_cast<typename E::SumW>(acc[i][j]));
        }
}

template <int DT>
void launchMatmulSimt(const LaunchContext& ctx, const void* a, uint64_t ars, uint64_t acs, const void* b, uint64_t brs, uint64_t bcs,
                      void* c, uint64_t m, uint64_t n, uint64_t k)
{
    typedef typename Elem<DT>::S S;
    dim3 grid(static_cast<unsigned int>((n + 63) / 64), static_cast<unsigned int>((m + 63) / 64));
    matmulSimtKernel<DT><<<grid, 256, 0, ctx.stream>>>(static_cast<const S*>(a), ars, acs, static_cast<const S*>(b), brs, bcs,
                                                       static_cast<S*>(c), m, n, k);
    if (ctx.launches) ++*ctx.launches;
}

// ---- data movement ----------------------------------------------------------------------------------------------
// transpose (aixDeviceCPU.cpp:391-405): element i of the dense source goes to the swapped coordinates in the result.
template <class S>
__global__ void __launch_bounds__(kBlock) transposeKernel(const S* __restrict__ src, S* __restrict__ dst, uint64_t count, Layout srcCanonical,
                                                          Layout dstStrides, int dim0, int dim1)
{
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        uint64_t coords[MAX_RANK], rem = i;
        for (int d = 0; d < srcCanonical.rank; ++d) { coords[d] = rem / srcCanonical.strides[d]; rem -= coords[d] * srcCanonical.strides[d]; }
        const uint64_t t = coords[dim0]; coords[dim0] = coords[dim1]; coords[dim1] = t;
        uint64_t off = 0;
        for (int d = 0; d < srcCanonical.rank; ++d) off += coords[d] * dstStrides.strides[d];
        dst[off] = src[i];
    }
}

// The same permutation for the case that matters at size: both tensors dense, nothing behind the second swapped dimension.
// The source is [A][X][B][Y], the result [A][Y][B][X]. A CTA moves a 64 x 64 tile of the (x, y) plane of one (a, b) through
// shared memory: rows of y are read with consecutive threads along y, rows of x are written with consecutive threads along x,
// so both sides of the copy touch whole lines instead of one element per line, and every thread has 16 independent loads
// in flight before the barrier.
constexpr uint32_t kTransposeTile = 64;
template <class S>
__global__ void __launch_bounds__(256) transposeTiledKernel(const S* __restrict__ src, S* __restrict__ dst, uint32_t A, uint32_t X, uint32_t B, uint32_t Y,
                                                            uint32_t tilesX, uint32_t tilesY, uint64_t tiles)
{
    __shared__ S tile[kTransposeTile][kTransposeTile + 1];
    const uint32_t tx = threadIdx.x & 63u, ty = threadIdx.x >> 6;      // 64 x 4 threads
    for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x)
    {
        uint64_t rest = t;
        const uint32_t tileY = static_cast<uint32_t>(rest % tilesY); rest /= tilesY;
        const uint32_t tileX = static_cast<uint32_t>(rest % tilesX); rest /= tilesX;
        const uint32_t b = static_cast<uint32_t>(rest % B);
        const uint32_t a = static_cast<uint32_t>(rest / B);
        const uint32_t x0 = tileX * kTransposeTile, y0 = tileY * kTransposeTile;
        const S* from = src + ((static_cast<uint64_t>(a) * X + x0) * B + b) * Y + y0;
        S* to = dst + ((static_cast<uint64_t>(a) * Y + y0) * B + b) * X + x0;
        const uint64_t fromPitch = static_cast<uint64_t>(B) * Y, toPitch = static_cast<uint64_t>(B) * X;
        const uint32_t limitX = min(kTransposeTile, X - x0), limitY = min(kTransposeTile, Y - y0);
        #pragma unroll
        for (uint32_t r = 0; r < kTransposeTile / 4; ++r)
        {
            const uint32_t x = ty + r * 4;
            if (x < limitX && tx < limitY) tile[x][tx] = from[x * fromPitch + tx];
        }
        __syncthreads();
        #pragma unroll
        for (uint32_t r = 0; r < kTransposeTile / 4; ++r)
        {
            const uint32_t y = ty + r * 4;
            if (tx < limitX && y < limitY) to[y * toPitch + tx] = tile[tx][y];
        }
        __syncthreads();
    }
}

// The same tile walk for 4-byte elements whose rows hold a whole number of 16-byte packs on both sides: the tile is read
// and written with 16-byte accesses (a quarter of the global load / store instructions), and transposed through scalar
// shared-memory accesses in between.
__global__ void __launch_bounds__(256) transposeTiledPackedKernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, uint32_t A, uint32_t X,
                                                                  uint32_t B, uint32_t Y, uint32_t tilesX, uint32_t tilesY, uint64_t tiles)
{
    __shared__ uint32_t tile[kTransposeTile][kTransposeTile + 1];
    const uint32_t part = threadIdx.x & 15u, line = threadIdx.x >> 4;      // 16 packs across a tile row, 16 rows per trip
    for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x)
    {
        uint64_t rest = t;
        const uint32_t tileY = static_cast<uint32_t>(rest % tilesY); rest /= tilesY;
        const uint32_t tileX = static_cast<uint32_t>(rest % tilesX); rest /= tilesX;
        const uint32_t b = static_cast<uint32_t>(rest % B);
        const uint32_t a = static_cast<uint32_t>(rest / B);
        const uint32_t x0 = tileX * kTransposeTile, y0 = tileY * kTransposeTile;
        const uint32_t* from = src + ((static_cast<uint64_t>(a) * X + x0) * B + b) * Y + y0;
        uint32_t* to = dst + ((static_cast<uint64_t>(a) * Y + y0) * B + b) * X + x0;
        const uint64_t fromPitch = static_cast<uint64_t>(B) * Y, toPitch = static_cast<uint64_t>(B) * X;
        const uint32_t limitX = min(kTransposeTile, X - x0), limitY = min(kTransposeTile, Y - y0);      // multiples of 4
        #pragma unroll
        for (uint32_t r = 0; r < kTransposeTile / 16; ++r)
        {
            const uint32_t x = line + r * 16, y = part * 4;
            if (x < limitX && y < limitY)
            {
                const uint4 pack = *reinterpret_cast<const uint4*>(from + x * fromPitch + y);
                tile[x][y] = pack.x; tile[x][y + 1] = pack.y; tile[x][y + 2] = pack.z; tile[x][y + 3] = pack.w;
            }
        }
        __syncthreads();
        #pragma unroll
        for (uint32_t r = 0; r < kTransposeTile / 16; ++r)
        {
            const uint32_t y = line + r * 16, x = part * 4;
            if (x < limitX && y < limitY)
                *reinterpret_cast<uint4*>(to + y * toPitch + x) = make_uint4(tile[x][y], tile[x + 1][y], tile[x + 2][y], tile[x + 3][y]);
        }
        __syncthreads();
    }
}

// sliceSet (aixDeviceCPU.cpp:470-499)
template <class S>
__global__ void __launch_bounds__(kBlock) sliceSetKernel(const S* __restrict__ src, Layout srcLayout, S* __restrict__ dst, Layout dstLayout,
                                                         uint64_t count, int dim, uint64_t start, uint64_t step, uint64_t sliceExtent)
{
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        uint64_t rem = i, off = 0;
        for (int d = dstLayout.rank - 1; d >= 0; --d)
        {
            const uint64_t extent = (d == dim) ? sliceExtent : dstLayout.shape[d];
            const uint64_t coord = rem % extent;
            rem /= extent;
            off += ((d == dim) ? (start + coord * step) : coord) * dstLayout.strides[d];
        }
        dst[off] = src[layoutOffset(i, srcLayout)];
    }
}

// tril / triu (aixDeviceCPU.cpp:565-622)
template <class S>
__global__ void __launch_bounds__(kBlock) triangleKernel(const S* __restrict__ src, Layout srcLayout, S* __restrict__ dst, Layout dstLayout,
                                                         uint64_t count, uint64_t rows, uint64_t cols, int64_t diagonal, bool lower)
{
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        const int64_t row = static_cast<int64_t>((i / cols) % rows), col = static_cast<int64_t>(i % cols);
        const bool zero = lower ? (col > row + diagonal) : (col < row + diagonal);
        dst[layoutOffset(i, dstLayout)] = zero ? S(0) : src[layoutOffset(i, srcLayout)];
    }
}

// tril / triu of dense tensors whose rows hold a whole number of 16-byte packs: one pack per thread and trip, the row and
// column of its first element found with one division, elements on the wrong side of the diagonal replaced by zero.
template <class S>
__global__ void __launch_bounds__(kBlock) trianglePackedKernel(const uint4* __restrict__ src, uint4* __restrict__ dst, uint64_t packs, uint32_t rows,
                                                               uint32_t packsPerRow, int64_t diagonal, bool lower)
{
    constexpr int kPer = 16 / sizeof(S);
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < packs; i += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        const uint64_t line = i / packsPerRow;
        const int64_t row = static_cast<int64_t>(line % rows), col0 = static_cast<int64_t>(i - line * packsPerRow) * kPer;
        // the pack's columns are col0 .. col0 + kPer - 1; kept when col <= row + diagonal (lower) or col >= row + diagonal (upper)
        const int64_t edge = row + diagonal;
        const bool allZero = lower ? (col0 > edge) : (col0 + kPer - 1 < edge);
        uint4 pack = make_uint4(0, 0, 0, 0);
        if (!allZero)
        {
            pack = src[i];
            S* e = reinterpret_cast<S*>(&pack);
            #pragma unroll
            for (int q = 0; q < kPer; ++q)
                if (lower ? (col0 + q > edge) : (col0 + q < edge)) e[q] = S(0);
        }
        dst[i] = pack;
    }
}

// indexSelect (aixDeviceCPU.cpp:502-531). An index outside [0, extent of the selected dimension) is not followed: the
// element is skipped (its destination keeps what it held) and *badIndex is raised, which the next synchronize() reports
// as an invalid argument. The reference's front end rejects such indices on the host before the device sees them
// (aixCore.hpp:1242, 1640-1650); callers of the C ABI have no such guard.
template <class S>
__global__ void __launch_bounds__(kBlock) indexSelectKernel(const S* __restrict__ src, Layout srcLayout, S* __restrict__ dst,
                                                            const int32_t* __restrict__ indices, Layout indexLayout, uint64_t indexCount,
                                                            uint64_t sliceSize, uint64_t dimSize, uint64_t dstCount, uint32_t* badIndex)
{
    const uint64_t extent = sliceSize ? dimSize / sliceSize : 0;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < dstCount; i += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        const uint64_t within = i % sliceSize, idx = (i / sliceSize) % indexCount, outer = i / (indexCount * sliceSize);
        const int64_t index = indices[layoutOffset(idx, indexLayout)];
        if (index < 0 || static_cast<uint64_t>(index) >= extent) { *badIndex = 1u; continue; }
        const uint64_t srcFlat = outer * dimSize + static_cast<uint64_t>(index) * sliceSize + within;
        dst[i] = src[layoutOffset(srcFlat, srcLayout)];
    }
}

// indexAdd (aixDeviceCPU.cpp:534-562). Several source slices may land on the same destination slice, so the kernel
// is parallel over (outer, within) and sequential over the index list: same order as the reference, no atomics.
// Out-of-range indices are skipped and reported like in indexSelect.
template <int DT>
__global__ void __launch_bounds__(kBlock) indexAddKernel(const typename Elem<DT>::S* __restrict__ src, Layout srcLayout,
                                                         typename Elem<DT>::S* __restrict__ dst, const int32_t* __restrict__ indices,
                                                         Layout indexLayout, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize,
                                                         uint64_t lanes, uint32_t* badIndex)
{
    typedef Reduce<DT, false> R;
    const uint64_t extent = sliceSize ? dimSize / sliceSize : 0;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; t < lanes; t += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        const uint64_t within = t % sliceSize, outer = t / sliceSize;
        for (uint64_t idx = 0; idx < indexCount; ++idx)
        {
            const int64_t index = indices[layoutOffset(idx, indexLayout)];
            if (index < 0 || static_cast<uint64_t>(index) >= extent) { *badIndex = 1u; continue; }
            const uint64_t dstOff = outer * dimSize + static_cast<uint64_t>(index) * sliceSize + within;
            const uint64_t srcFlat = outer * indexCount * sliceSize + idx * sliceSize + within;
            dst[dstOff] = R::finish(R::merge(R::liftStored(dst[dstOff]), R::liftStored(src[layoutOffset(srcFlat, srcLayout)])));
        }
    }
}

// indexAdd with few (outer, within) lanes and a long index list: parallel over every source element, colliding
// destinations resolved by atomics (the reference's Metal kernels do the same, aixDeviceMetalShaders.hpp:2289-2314).
// Integer sums wrap, so any order gives the reference's bits; floating sums depend on the order of colliding adds within
// rounding. f32 / f64 / i32 / i64 use the native atomics; 16- and 8-bit types a compare-and-swap on the enclosing 32-bit
// word, rounding to the storage type after every add like the sequential form.
template <int DT> __device__ __forceinline__ void atomicAccumulate(typename Elem<DT>::S* dst, uint64_t off, typename Elem<DT>::S value)
{
    typedef Elem<DT> E;
    typedef typename E::S S;
    typedef Reduce<DT, false> R;
    if constexpr (DT == 0) atomicAdd(reinterpret_cast<double*>(dst) + off, static_cast<double>(value));
    else if constexpr (DT == 1) atomicAdd(reinterpret_cast<float*>(dst) + off, static_cast<float>(value));
    else if constexpr (DT == 4) atomicAdd(reinterpret_cast<unsigned long long*>(dst) + off, static_cast<unsigned long long>(value));
    else if constexpr (DT == 5) atomicAdd(reinterpret_cast<int*>(dst) + off, static_cast<int>(value));
    else
    {
        const uintptr_t address = reinterpret_cast<uintptr_t>(dst + off);
        unsigned int* word = reinterpret_cast<unsigned int*>(address & ~uintptr_t(3));
        const unsigned shift = static_cast<unsigned>(address & 3u) * 8u;
        const unsigned mask = (sizeof(S) == 2 ? 0xFFFFu : 0xFFu) << shift;
        unsigned int seen = *word, assumed;
        do
        {
            assumed = seen;
            S held;
            if constexpr (sizeof(S) == 2) { const uint16_t bits = static_cast<uint16_t>((assumed & mask) >> shift); memcpy(&held, &bits, 2); }
            else { const uint8_t bits = static_cast<uint8_t>((assumed & mask) >> shift); memcpy(&held, &bits, 1); }
            const S sum = R::finish(R::merge(R::liftStored(held), R::liftStored(value)));
            unsigned int bits = 0;
            memcpy(&bits, &sum, sizeof(S));
            seen = atomicCAS(word, assumed, (assumed & ~mask) | ((bits << shift) & mask));
        } while (seen != assumed);
    }
}

template <int DT>
__global__ void __launch_bounds__(kBlock) indexAddAtomicKernel(const typename Elem<DT>::S* __restrict__ src, Layout srcLayout,
                                                               typename Elem<DT>::S* dst, const int32_t* __restrict__ indices, Layout indexLayout,
                                                               uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t srcCount,
                                                               uint32_t* badIndex)
{
    const uint64_t extent = sliceSize ? dimSize / sliceSize : 0;
    for (uint64_t t = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; t < srcCount; t += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        const uint64_t within = t % sliceSize, idx = (t / sliceSize) % indexCount, outer = t / (indexCount * sliceSize);
        const int64_t index = indices[layoutOffset(idx, indexLayout)];
        if (index < 0 || static_cast<uint64_t>(index) >= extent) { *badIndex = 1u; continue; }
        atomicAccumulate<DT>(dst, outer * dimSize + static_cast<uint64_t>(index) * sliceSize + within, src[layoutOffset(t, srcLayout)]);
    }
}

template <int DT>
__global__ void __launch_bounds__(kBlock) scaleKernel(typename Elem<DT>::S* data, uint64_t count, double scale)
{
    typedef Elem<DT> E;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * kBlock)
    {
        if (DT == 0) data[i] = E::store(static_cast<typename E::V>(static_cast<double>(E::load(data[i])) * scale));
        else         data[i] = E::store(static_cast<typename E::V>(static_cast<float>(E::load(data[i])) * static_cast<float>(scale)));
    }
}

__global__ void __launch_bounds__(kBlock) flushL2Kernel(uint4* buffer, uint64_t count)
{
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < count; i += static_cast<uint64_t>(gridDim.x) * kBlock)
        buffer[i] = make_uint4(static_cast<unsigned>(i), 0u, 0u, 0u);
}

inline bool isCanonical(const Layout& l, const uint64_t* shape)
{
    uint64_t expect = 1;
    for (int d = l.rank - 1; d >= 0; --d)
    {
        if (shape[d] != 1 && l.strides[d] != expect) return false;
        expect *= shape[d];
    }
    return true;
}

template <int DT> void launchTranspose(const LaunchContext& ctx, const void* src, void* dst, uint64_t count, const Layout& sc, const Layout& ds, int d0, int d1)
{
    typedef typename Elem<DT>::S S;
    if (d0 > d1) std::swap(d0, d1);
    if (d0 != d1 && count >= 4096 && count < (uint64_t(1) << 40))
    {
        // source dense in its own shape, result dense in the swapped shape, second swapped dimension innermost (or followed by
        // dimensions of one element only): the tiled kernel
        uint64_t swapped[MAX_RANK];
        for (int d = 0; d < sc.rank; ++d) swapped[d] = sc.shape[d];
        std::swap(swapped[d0], swapped[d1]);
        uint64_t A = 1, B = 1, C = 1;
        for (int d = 0; d < d0; ++d) A *= sc.shape[d];
        for (int d = d0 + 1; d < d1; ++d) B *= sc.shape[d];
        for (int d = d1 + 1; d < sc.rank; ++d) C *= sc.shape[d];
        const uint64_t X = sc.shape[d0], Y = sc.shape[d1];
        if (C == 1 && isCanonical(sc, sc.shape) && isCanonical(ds, swapped) && A < (1u << 31) && B < (1u << 31) && X < (1u << 31) && Y < (1u << 31) && X >= 8 && Y >= 8)
        {
            const uint64_t tilesX = (X + kTransposeTile - 1) / kTransposeTile, tilesY = (Y + kTransposeTile - 1) / kTransposeTile, tiles = A * B * tilesX * tilesY;
            const unsigned grid = static_cast<unsigned>(std::min<uint64_t>(tiles, static_cast<uint64_t>(ctx.smCount) * 8));
            if (sizeof(S) == 4 && X % 4 == 0 && Y % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0)
            {
                transposeTiledPackedKernel<<<grid, 256, 0, ctx.stream>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), static_cast<uint32_t>(A),
                                                                        static_cast<uint32_t>(X), static_cast<uint32_t>(B), static_cast<uint32_t>(Y),
                                                                        static_cast<uint32_t>(tilesX), static_cast<uint32_t>(tilesY), tiles);
                return;
            }
            transposeTiledKernel<S><<<grid, 256, 0, ctx.stream>>>(static_cast<const S*>(src), static_cast<S*>(dst), static_cast<uint32_t>(A), static_cast<uint32_t>(X),
                                                                  static_cast<uint32_t>(B), static_cast<uint32_t>(Y), static_cast<uint32_t>(tilesX),
                                                                  static_cast<uint32_t>(tilesY), tiles);
            return;
        }
    }
    transposeKernel<S><<<gridFor(count, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), static_cast<S*>(dst), count, sc, ds, d0, d1);
}
// sliceSet between dense tensors: element i of the source is (outer, j, w) with w running over the dimensions behind the
// sliced one; it lands at ((outer * extent + start + j * step) * inner + w) - two divisions in the narrowest index type
// instead of a mixed-radix walk over both layouts.
template <class S, class I>
__global__ void __launch_bounds__(kBlock) sliceSetDenseKernel(const S* __restrict__ src, S* __restrict__ dst, I count, I inner, I sliceExtent,
                                                              uint64_t dimExtent, uint64_t start, uint64_t step)
{
    for (I i = static_cast<I>(blockIdx.x) * kBlock + threadIdx.x; i < count; i += static_cast<I>(gridDim.x) * kBlock)
    {
        const I q = i / inner, w = i - q * inner, outer = q / sliceExtent, j = q - outer * sliceExtent;
        dst[(static_cast<uint64_t>(outer) * dimExtent + start + static_cast<uint64_t>(j) * step) * inner + w] = src[i];
    }
}

template <int DT> void launchSliceSet(const LaunchContext& ctx, const void* src, const Layout& sl, void* dst, const Layout& dl, uint64_t count,
                                      int dim, uint64_t start, uint64_t step, uint64_t sliceExtent)
{
    typedef typename Elem<DT>::S S;
    if (count >= 4096 && sliceExtent > 0 && isCanonical(sl, sl.shape) && isCanonical(dl, dl.shape))
    {
        uint64_t inner = 1;
        for (int d = dim + 1; d < dl.rank; ++d) inner *= dl.shape[d];
        const unsigned grid = static_cast<unsigned>(std::min<uint64_t>((count + kBlock - 1) / kBlock, static_cast<uint64_t>(ctx.smCount) * 32));
        if (count < (uint64_t(1) << 32))
            sliceSetDenseKernel<S, uint32_t><<<grid, kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), static_cast<S*>(dst), static_cast<uint32_t>(count),
                                                                             static_cast<uint32_t>(inner), static_cast<uint32_t>(sliceExtent), dl.shape[dim], start, step);
        else
            sliceSetDenseKernel<S, uint64_t><<<grid, kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), static_cast<S*>(dst), count, inner, sliceExtent,
                                                                             dl.shape[dim], start, step);
        return;
    }
    sliceSetKernel<S><<<gridFor(count, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), sl, static_cast<S*>(dst), dl, count, dim, start, step, sliceExtent);
}
template <int DT> void launchTriangle(const LaunchContext& ctx, const void* src, const Layout& sl, void* dst, const Layout& dl, uint64_t count,
                                      uint64_t rows, uint64_t cols, int64_t diagonal, bool lower)
{
    typedef typename Elem<DT>::S S;
    constexpr uint64_t kPer = 16 / sizeof(S);
    if (cols % kPer == 0 && count >= 4096 && rows < (1ull << 32) && cols / kPer < (1ull << 32) && isCanonical(sl, sl.shape) && isCanonical(dl, dl.shape) &&
        reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0)
    {
        const uint64_t packs = count / kPer;
        trianglePackedKernel<S><<<gridFor(packs, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), packs, static_cast<uint32_t>(rows),
                                                                                       static_cast<uint32_t>(cols / kPer), diagonal, lower);
        return;
    }
    triangleKernel<S><<<gridFor(count, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), sl, static_cast<S*>(dst), dl, count, rows, cols, diagonal, lower);
}
// indexSelect from a dense source with a dense index list: every selected slice is one contiguous run of `runLength` units
// (16-byte packs when the slices allow it, elements otherwise), copied by the threads of a CTA side by side; a CTA takes
// the runs blockIdx.y, blockIdx.y + gridDim.y, ... One index load per run instead of two mixed-radix decompositions per element.
template <class V>
__global__ void __launch_bounds__(kBlock) indexSelectRunsKernel(const V* __restrict__ src, V* __restrict__ dst, const int32_t* __restrict__ indices,
                                                                uint64_t indexCount, uint64_t runLength, uint64_t extent, uint64_t runs, uint32_t* badIndex)
{
    for (uint64_t run = blockIdx.y; run < runs; run += gridDim.y)
    {
        const uint64_t outer = run / indexCount;
        const int64_t index = indices[run - outer * indexCount];
        if (index < 0 || static_cast<uint64_t>(index) >= extent)
        {
            if (threadIdx.x == 0 && blockIdx.x == 0) *badIndex = 1u;
            continue;
        }
        const V* from = src + (outer * extent + static_cast<uint64_t>(index)) * runLength;
        V* to = dst + run * runLength;
        for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < runLength; i += static_cast<uint64_t>(gridDim.x) * kBlock) to[i] = from[i];
    }
}

template <int DT> void launchIndexSelect(const LaunchContext& ctx, const void* src, const Layout& sl, void* dst, const int32_t* indices,
                                         const Layout& il, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t dstCount)
{
    typedef typename Elem<DT>::S S;
    const bool denseIndices = il.rank == 0 || (il.rank == 1 && (il.strides[0] == 1 || il.shape[0] == 1));
    if (denseIndices && sliceSize >= 32 && indexCount > 0 && dstCount >= 4096 && isCanonical(sl, sl.shape))
    {
        const uint64_t extent = dimSize / sliceSize, runs = dstCount / sliceSize;
        const bool packs = (sliceSize * sizeof(S)) % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
        const uint64_t runLength = packs ? sliceSize * sizeof(S) / 16 : sliceSize;
        const dim3 grid(static_cast<unsigned>(std::min<uint64_t>((runLength + kBlock - 1) / kBlock, 16)),
                        static_cast<unsigned>(std::min<uint64_t>(runs, static_cast<uint64_t>(ctx.smCount) * 32)));
        if (packs)
            indexSelectRunsKernel<uint4><<<grid, kBlock, 0, ctx.stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), indices, indexCount,
                                                                         runLength, extent, runs, badIndexWord(ctx));
        else
            indexSelectRunsKernel<S><<<grid, kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), static_cast<S*>(dst), indices, indexCount, runLength, extent,
                                                                     runs, badIndexWord(ctx));
        return;
    }
    indexSelectKernel<S><<<gridFor(dstCount, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), sl, static_cast<S*>(dst), indices, il,
                                                                                   indexCount, sliceSize, dimSize, dstCount, badIndexWord(ctx));
}
// The atomic form for a dense source with a dense index list: a source slice is one contiguous run, added to the run it
// selects by the threads of a CTA side by side - one index load and one address computation per run instead of a mixed-radix
// walk per element.
template <int DT>
__global__ void __launch_bounds__(kBlock) indexAddRunsKernel(const typename Elem<DT>::S* __restrict__ src, typename Elem<DT>::S* __restrict__ dst,
                                                             const int32_t* __restrict__ indices, uint64_t indexCount, uint64_t sliceSize, uint64_t extent,
                                                             uint64_t runs, uint32_t* badIndex)
{
    for (uint64_t run = blockIdx.y; run < runs; run += gridDim.y)
    {
        const uint64_t outer = run / indexCount;
        const int64_t index = indices[run - outer * indexCount];
        if (index < 0 || static_cast<uint64_t>(index) >= extent)
        {
            if (threadIdx.x == 0 && blockIdx.x == 0) *badIndex = 1u;
            continue;
        }
        const typename Elem<DT>::S* from = src + run * sliceSize;
        const uint64_t base = (outer * extent + static_cast<uint64_t>(index)) * sliceSize;
        for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kBlock + threadIdx.x; i < sliceSize; i += static_cast<uint64_t>(gridDim.x) * kBlock)
            atomicAccumulate<DT>(dst, base + i, from[i]);
    }
}

template <int DT> void launchIndexAdd(const LaunchContext& ctx, const void* src, const Layout& sl, void* dst, const int32_t* indices,
                                      const Layout& il, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t srcCount)
{
    typedef typename Elem<DT>::S S;
    const uint64_t lanes = indexCount ? srcCount / indexCount : 0;
    if (lanes == 0) return;
    // Enough (outer, within) lanes to fill the GPU: one thread per lane walks the index list in order (deterministic,
    // coalesced). Fewer lanes and a longer list: one thread per source element with atomics.
    static const bool atomicsAllowed = []{ const char* v = std::getenv("AIXB200_INDEX_ADD_ATOMICS"); return !(v && v[0] == '0'); }();
    if (atomicsAllowed && lanes < static_cast<uint64_t>(ctx.smCount) * 512 && indexCount >= 8)
    {
        const bool denseIndices = il.rank == 0 || (il.rank == 1 && (il.strides[0] == 1 || il.shape[0] == 1));
        if (denseIndices && sliceSize >= 32 && srcCount >= 4096 && isCanonical(sl, sl.shape))
        {
            const uint64_t runs = srcCount / sliceSize;
            const dim3 grid(static_cast<unsigned>(std::min<uint64_t>((sliceSize + kBlock - 1) / kBlock, 16)),
                            static_cast<unsigned>(std::min<uint64_t>(runs, static_cast<uint64_t>(ctx.smCount) * 32)));
            indexAddRunsKernel<DT><<<grid, kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), static_cast<S*>(dst), indices, indexCount, sliceSize,
                                                                    dimSize / sliceSize, runs, badIndexWord(ctx));
            return;
        }
        indexAddAtomicKernel<DT><<<gridFor(srcCount, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), sl, static_cast<S*>(dst), indices, il,
                                                                                          indexCount, sliceSize, dimSize, srcCount, badIndexWord(ctx));
        return;
    }
    indexAddKernel<DT><<<gridFor(lanes, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<const S*>(src), sl, static_cast<S*>(dst), indices, il,
                                                                                 indexCount, sliceSize, dimSize, lanes, badIndexWord(ctx));
}
template <int DT> void launchScale(const LaunchContext& ctx, void* data, uint64_t count, double scale)
{
    scaleKernel<DT><<<gridFor(count, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<typename Elem<DT>::S*>(data), count, scale);
}

}   // namespace

void argmaxAll(const LaunchContext& ctx, const View& src, int32_t* dst, bool oneHot, uint64_t count)
{
    AIXB200_DISPATCH_DTYPE(src.dtype, launchArgmaxAll, ctx, src, dst, oneHot, count);
}

void argmaxAlong(const LaunchContext& ctx, uint32_t dtype, const void* src, const ReduceDim* dims, int rank, int reducedDim,
                 int32_t* dst, bool oneHot, uint64_t)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchArgmaxAlong, ctx, src, dims, rank, reducedDim, dst, oneHot);
}

void matmulSimt(const LaunchContext& ctx, uint32_t dtype, const void* a, uint64_t ars, uint64_t acs, const void* b, uint64_t brs,
                uint64_t bcs, void* c, uint64_t m, uint64_t n, uint64_t k)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchMatmulSimt, ctx, a, ars, acs, b, brs, bcs, c, m, n, k);
}

void transposeGeneral(const LaunchContext& ctx, uint32_t dtype, const void* src, void* dst, uint64_t count, const Layout& sc,
                      const Layout& ds, int dim0, int dim1)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchTranspose, ctx, src, dst, count, sc, ds, dim0, dim1);
    if (ctx.launches) ++*ctx.launches;
}

void sliceSet(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& sl, void* dst, const Layout& dl, uint64_t count,
              int dim, uint64_t start, uint64_t step, uint64_t sliceExtent)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchSliceSet, ctx, src, sl, dst, dl, count, dim, start, step, sliceExtent);
    if (ctx.launches) ++*ctx.launches;
}

void triangle(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& sl, void* dst, const Layout& dl, uint64_t count,
              uint64_t rows, uint64_t cols, int64_t diagonal, bool lower)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchTriangle, ctx, src, sl, dst, dl, count, rows, cols, diagonal, lower);
    if (ctx.launches) ++*ctx.launches;
}

void indexSelect(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& sl, void* dst, const int32_t* indices,
                 const Layout& il, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t dstCount)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchIndexSelect, ctx, src, sl, dst, indices, il, indexCount, sliceSize, dimSize, dstCount);
    if (ctx.launches) ++*ctx.launches;
}

void indexAdd(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& sl, void* dst, const int32_t* indices,
              const Layout& il, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t srcCount)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchIndexAdd, ctx, src, sl, dst, indices, il, indexCount, sliceSize, dimSize, srcCount);
    if (ctx.launches) ++*ctx.launches;
}

void scaleInPlace(const LaunchContext& ctx, uint32_t dtype, void* data, uint64_t count, double scale)
{
    AIXB200_DISPATCH_DTYPE(dtype, launchScale, ctx, data, count, scale);
    if (ctx.launches) ++*ctx.launches;
}

void flushL2(const LaunchContext& ctx, void* buffer, size_t bytes)
{
    const uint64_t count = bytes / 16;
    flushL2Kernel<<<gridFor(count, ctx.smCount), kBlock, 0, ctx.stream>>>(static_cast<uint4*>(buffer), count);
    if (ctx.launches) ++*ctx.launches;
}

}   // namespace aixb200::kernels
