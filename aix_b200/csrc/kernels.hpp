// Host-callable launchers of the fixed (ahead-of-time compiled) sm_100a kernels.
#pragma once

#include "common.hpp"

typedef struct CUstream_st* cudaStream_t;

namespace aixb200::kernels
{

struct LaunchContext
{
    cudaStream_t stream;
    int          smCount;
    void*        scratch;        // device scratch, zero-initialised once; kernels leave its counters at zero
    size_t       scratchBytes;
    uint64_t*    launches;       // incremented once per kernel launch
    uint32_t*    gemmLaunches = nullptr;   // host counter of tensor-core matmul launches that used this scratch block's tile scheduler
};

// Layout of the scratch block shared by the reduction kernels.
constexpr size_t kScratchCounterBytes = 256;        // ticket counters at the start
constexpr size_t kScratchTimeoutOffset  = 128;      // raised by a kernel whose bounded wait ran out
constexpr size_t kScratchBadIndexOffset = 132;      // raised by indexSelect / indexAdd on an index outside the dimension
constexpr size_t kMaxReduceBlocks     = 4096;       // upper bound of partials a full reduction may write
// The device allocates this much beyond LaunchContext::scratchBytes: counters of the tensor-core matmul's split tiles.
constexpr size_t kGemmCounterBytes    = 4096 + 16384;
// ... and, behind the first 4096 bytes, the tile scheduler of the CTA-pair matmul: eight rotating tile counters (64 bytes
// apart) and, from kGemmRingOffset on, a ring of 16 published tile indices (8 bytes each) per cluster.
constexpr size_t kGemmSchedulerOffset = 4096;
constexpr size_t kGemmRingOffset      = 4096 + 512;
constexpr size_t kGemmRingSlots       = 16;

// ---- full reductions (Device::sum / Device::max, aixDevice.hpp:52,60) -----------------------------------------
// dst[0] = sum or max of all elements of src, in src's element type.
void reduceAll(const LaunchContext& ctx, bool isMax, const View& src, void* dst);
// Same kernel with caller-provided scratch (partials + ticket counter).
void reduceAllWithScratch(const LaunchContext& ctx, bool isMax, const View& src, void* dst, void* scratch, size_t scratchBytes);
// Sum with the scratch in a static __device__ array of the library (no allocation anywhere on the path).
// Inputs above kStaticScratchMaxElements are refused by the caller. Returns a CUDA error string or nullptr.
constexpr uint64_t kStaticScratchMaxElements = uint64_t(1) << 30;
constexpr size_t   kStaticScratchBytes = 32768;
const char* sumWithStaticScratch(const LaunchContext& ctx, int ordinal, const View& src, void* dst);

// ---- partial reductions (Device::reduceTo / maxTo, aixDevice.hpp:70-71) ----------------------------------------
// One (extent, source stride, kept?) triple per collapsed source dimension, outermost first. Kept dimensions index
// the dense destination in row-major order; the others are folded with + or max INTO the destination.
struct ReduceDim { uint64_t extent; uint64_t stride; bool kept; };
void reduceInto(const LaunchContext& ctx, bool isMax, uint32_t dtype, const void* src, const ReduceDim* dims, int rank, void* dst);

// ---- argmax family (aixDevice.hpp:61-62, 72-73) ----------------------------------------------------------------
void argmaxAll(const LaunchContext& ctx, const View& src, int32_t* dst, bool oneHot, uint64_t count);
void argmaxAlong(const LaunchContext& ctx, uint32_t dtype, const void* src, const ReduceDim* dims, int rank, int reducedDim,
                 int32_t* dst, bool oneHot, uint64_t srcCount);

// ---- matmul fallback on CUDA cores (any element type, any 2-D strides) ------------------------------------------
void matmulSimt(const LaunchContext& ctx, uint32_t dtype, const void* a, uint64_t aRowStride, uint64_t aColStride,
                const void* b, uint64_t bRowStride, uint64_t bColStride, void* c, uint64_t m, uint64_t n, uint64_t k);

// ---- data movement (aixDevice.hpp:64, 74-81) -------------------------------------------------------------------
struct Layout { int rank; uint64_t shape[MAX_RANK]; uint64_t strides[MAX_RANK]; };
void transposeGeneral(const LaunchContext& ctx, uint32_t dtype, const void* src, void* dst, uint64_t count,
                      const Layout& srcCanonical, const Layout& dstStrides, int dim0, int dim1);
void sliceSet(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& srcLayout, void* dst,
              const Layout& dstLayout, uint64_t count, int dim, uint64_t start, uint64_t step, uint64_t sliceExtent);
void triangle(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& srcLayout, void* dst,
              const Layout& dstLayout, uint64_t count, uint64_t rows, uint64_t cols, int64_t diagonal, bool lower);
void indexSelect(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& srcLayout, void* dst, const int32_t* indices,
                 const Layout& indexLayout, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t dstCount);
void indexAdd(const LaunchContext& ctx, uint32_t dtype, const void* src, const Layout& srcLayout, void* dst, const int32_t* indices,
              const Layout& indexLayout, uint64_t indexCount, uint64_t sliceSize, uint64_t dimSize, uint64_t srcCount);
void scaleInPlace(const LaunchContext& ctx, uint32_t dtype, void* data, uint64_t count, double scale);
void flushL2(const LaunchContext& ctx, void* buffer, size_t bytes);

}   // namespace aixb200::kernels
