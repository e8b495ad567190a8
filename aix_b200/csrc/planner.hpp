// Lazy op recorder and fusion planner.
//
// Re-creates the job of the reference's fuse::FuseEngine (aixFuse.hpp:166-217, aixFuse.cpp:89-1014) with a
// different algorithm. The reference grows subgraphs by breadth-first search over a dependency DAG keyed by
// (pointer, dtype, offset); here every recorded op is placed, in program order, into the latest *open kernel group*
// that (a) iterates over the same number of elements and (b) lies at or after every group the op depends on.
// Dependencies are found on byte ranges of the storages, so views of one storage with different offsets or
// strides are ordered correctly:
//   * an input that is element-for-element the output of an earlier op in the same group is taken from a register;
//   * any other overlap (a transposed or shifted view of something written earlier, a write into something read
//     earlier through a different view) forces a later kernel, because it needs a grid-wide barrier;
//   * a fill of a one-element tensor that is later read through an all-zero-stride broadcast view becomes a kernel
//     scalar of the reader (what the reference achieves with absorbed fills, aixFuse.cpp:552-576, 693-710).
// A full sum or max whose operand is produced by a pending op joins that op's kernel as a reduction epilogue (the
// reference ends the fused region at every reduction, aixDeviceMetal.cpp:296-359): the operand is folded while it is
// still in registers, and if its storage is already dead it never reaches memory. The one-element result is written
// when the whole grid has finished, so every other access to it is ordered into a later (or earlier) kernel.
// A result whose storage has already been deallocated and whose readers all sit in the same group is never
// written to memory (the reference's dead-intermediate elision, aixFuse.cpp:538-550).
#pragma once

#include "common.hpp"

#include <string>
#include <unordered_set>
#include <vector>

namespace aixb200
{

enum class Op : uint8_t { Add, Sub, Mul, Div, Neg, Sqrt, Sin, Cos, Tanh, Log, Exp, Pow, Fill, Cast,
                          SumAll, MaxAll,   // full reductions recorded behind a pending producer: in[0] -> one element
                          SumRows, MaxRows, // reductions over the trailing dimension of a dense [rows, cols] operand recorded behind
                                            // its pending producer: in[0] = operand, in[1] = out = the `rows` results, which
                                            // accumulate into what the destination holds (reduceTo / maxTo contract)
                          COUNT };
inline bool isRowReduction(Op op) { return op == Op::SumRows || op == Op::MaxRows; }
inline bool isReduction(Op op) { return op == Op::SumAll || op == Op::MaxAll || isRowReduction(op); }
const char* opName(Op op);

struct OpRecord
{
    Op         op;
    uint8_t    numInputs = 0;
    View       in[2];
    View       out;
    ScalarBits scalar{};       // Fill: the value, already converted to out.dtype
    uint64_t   rowCols = 0;    // SumRows / MaxRows: length of a row of in[0]
};

// How element i of the iteration space maps to an element of a view.
enum class Access : uint8_t
{
    Dense,      // offset + i
    Scalar,     // offset                       (one element broadcast everywhere)
    RowBcast,   // offset + (i % cols)          (a row vector broadcast down the rows; stride (0,1))
    ColBcast,   // offset + (i / cols) * stride (a column vector broadcast along the rows; stride (s,0))
    General,    // mixed-radix decomposition of i over the collapsed shape
};

struct OperandRef
{
    enum Kind : uint8_t { None, Reg, Load } kind = None;
    uint16_t index = 0;        // node index (Reg) or load index (Load)
};

struct KernelNode
{
    Op         op;
    uint8_t    dtype;          // element type the op computes in (its result type)
    uint8_t    srcDtype;       // Cast: element type of the operand
    OperandRef a, b;
    uint16_t   scalarIndex = 0;   // Fill: index into KernelSpec::scalars
};

struct KernelLoad  { View view; Access access; };
struct KernelReduce { uint16_t node; bool isMax; uint8_t dtype; View out; bool absBits = false; };   // out: the one-element result;
                                            // absBits (f32 only): the result is the bit pattern of max|x| (a matmul operand's scale)
struct KernelStore { View view; Access access; uint16_t node; };
// One result per row of the kernel's [count / rowCols, rowCols] iteration space: out[row] = fold(initial, node over the row).
// The initial value is what the destination holds, or - when the destination was filled by a pending op that nobody
// else reads - that fill's value as a kernel scalar (the fill itself is then never stored).
struct KernelRowReduce { uint16_t node; bool isMax; uint8_t dtype; View out; bool initImmediate; uint16_t scalarIndex; };

// One fused kernel: loads, straight-line nodes, stores, all over `count` elements.
struct KernelSpec
{
    uint64_t                 count = 0;
    std::vector<KernelLoad>  loads;
    std::vector<KernelNode>  nodes;
    std::vector<KernelStore> stores;
    std::vector<KernelReduce> reductions;  // folded over all `count` elements of a node
    std::vector<KernelRowReduce> rowReductions;   // folded over each row of rowCols elements
    uint64_t                 rowCols = 0;  // non-zero: the kernel walks the elements row by row (one warp or CTA per row)
    std::vector<ScalarBits>  scalars;      // runtime values; not part of the kernel's identity
    std::vector<uint8_t>     scalarDtypes;
    uint32_t                 opsFolded = 0;    // recorded ops this kernel stands for
    uint32_t                 storesElided = 0;
    uint32_t                 fillsAbsorbed = 0;
};

struct PlannerLimits
{
    size_t maxTensorsPerKernel = 24;   // loads + stores
    size_t maxNodesPerKernel   = 160;
    size_t maxReductionsPerKernel = 4;
    bool   fusion              = true;
};

Access classifyAccess(const View& v, uint64_t count);

// Plans `ops` (program order). `released` holds the storage bases that were deallocated while these ops were
// pending: nothing after this batch can read them.
std::vector<KernelSpec> planKernels(const std::vector<OpRecord>& ops, const std::unordered_set<const void*>& released,
                                    const PlannerLimits& limits);

}   // namespace aixb200
