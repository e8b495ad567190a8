// CUDA C generator for fused elementwise kernels.
//
// Counterpart of the reference's Metal-source generator (aixDeviceMetalKernelGen.cpp:480-710): one straight-line
// SSA statement per op, one kernel per fused group, runtime scalars passed as arguments so that kernels are shared
// between expressions that differ only in constants (aixDeviceMetalKernelGen.cpp:421-478). What differs is the
// kernel shape, which is written for B200: every thread moves 16-byte packs with 128-bit loads and stores, walks the
// tensor with a grid-stride loop, keeps several packs in flight, and carries broadcast row/column indices
// incrementally instead of re-deriving them with a division per access.
#pragma once

#include "planner.hpp"

#include <string>
#include <vector>

namespace aixb200
{

struct CodegenOptions
{
    bool strictMath = true;   // reported in the key only; the compile flags are chosen by the caller
    int  block      = 256;    // threads per CTA
    int  unroll     = 2;      // packs in flight per thread
    int  rowMinBlocks = -1;   // row-form kernels: CTAs per SM asked for in __launch_bounds__ (0: left to the compiler). -1: automatic -
                              // 16-bit row-form kernels ask for 8 and keep one pack in flight per thread (measured on the
                              // broadcast + reduction configuration, bf16 8192 x 8192: 63 us against 68 us), others ask for nothing
};

// Everything that selects a distinct kernel for one KernelSpec at launch time.
struct KernelVariant
{
    int      vec = 1;          // elements per pack (16 bytes of the narrowest element type)
    bool     packed16 = false; // one f16/bf16 type throughout: two elements per register on the packed pipes
    bool     index64 = false;  // element count does not fit 32 bits
    bool     rowMode = false;  // the kernel walks [count / rowCols, rowCols] row by row and folds per-row results
    bool     warpPerRow = false; // rowMode: one warp per row (short rows, many of them) instead of one CTA per row
    uint32_t fastLoads = 0;    // bit l: load l may use the wide / hoisted path
    uint32_t fastStores = 0;   // bit s: store s may use 128-bit stores
};

KernelVariant chooseVariant(const KernelSpec& spec);

// Identity of the generated code: two (spec, variant) pairs with equal keys generate identical source.
std::string kernelKey(const KernelSpec& spec, const KernelVariant& variant, const CodegenOptions& options);

std::string generateKernelSource(const KernelSpec& spec, const KernelVariant& variant, const CodegenOptions& options,
                                 const std::string& entryName);

// Kernel argument block (an array of 64-bit slots) in the order the generated kernel expects. `scratch` is the
// device scratch block (tickets in its first bytes, 64-bit partials from kReductionPartialsOffset on); only kernels
// with reductions use it.
constexpr size_t kReductionPartialsOffset = 256;
constexpr size_t kReductionMaxBlocks = 4096;       // partials per reduction: the launch grid is capped to this
std::vector<uint64_t> packKernelArguments(const KernelSpec& spec, const KernelVariant& variant, void* scratch);

}   // namespace aixb200
