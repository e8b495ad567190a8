// The B200 device object behind the C ABI: CUDA context and stream, allocator, lazy recorder, kernel cache.
// Counterpart of the reference's DeviceMetal (aixDeviceMetal.hpp / .cpp), rebuilt around CUDA's model:
// one in-order stream instead of command buffers, NVRTC + cubin cache instead of MTL libraries, stream-ordered
// block reuse instead of completion handlers.
#pragma once

#include "allocator.hpp"
#include "codegen.hpp"
#include "planner.hpp"
#include "scalar.hpp"

#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

typedef struct CUstream_st* cudaStream_t;
typedef struct CUevent_st* cudaEvent_t;
typedef struct CUfunc_st* CUfunction;
typedef struct CUmod_st* CUmodule;

namespace aixb200
{

class Comm;

struct CompiledKernel
{
    CUmodule   module = nullptr;
    CUfunction function = nullptr;
    int        residentPerSm = 0;     // CTAs of this kernel that fit on one SM at once (0: unknown)
    std::string source;
};

class Device
{
public:
    explicit Device(const aixb200_config& cfg);
    ~Device();
    Device(const Device&) = delete;
    Device& operator=(const Device&) = delete;

    const std::string& name() const { return m_name; }
    bool dryRun() const { return m_cfg.dry_run != 0; }
    cudaStream_t stream() const { return m_stream; }
    int ordinal() const { return m_cfg.ordinal; }
    int smCount() const { return m_smCount; }

    // memory
    void* allocate(size_t bytes);
    void  deallocate(void* p);
    void  emptyCache();
    void  synchronize();

    // recorded elementwise ops
    void recordBinary(Op op, const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r, const char* what);
    void recordUnary(Op op, const aixb200_tensor* a, const aixb200_tensor* r, const char* what);
    void recordFill(const void* scalar, uint32_t scalarDtype, const aixb200_tensor* r);
    void recordFillMin(const aixb200_tensor* r);
    bool recordReduction(Op op, const View& src, const View& dst);
    bool recordRowReduction(bool isMax, const View& src, const View& dst, uint64_t rows, uint64_t cols);
    // Emits the recorded ops. A fill that nothing else in the batch touches, whose storage is alive and which the call in
    // progress does not touch either stays recorded (the reference keeps such fills deferred too, aixFuse.cpp:891-916):
    // the op that eventually uses the buffer - typically an in-place accumulation a few matmuls later - then absorbs it.
    // flushAll() emits everything (synchronize, event records, memory pressure).
    void flush(bool keepIdleFills = true);
    void flushAll() { flush(false); }

    // immediate ops (flush first, then launch fixed kernels)
    void sum(const aixb200_tensor* a, const aixb200_tensor* r);
    void max(const aixb200_tensor* a, const aixb200_tensor* r);
    void sumStaticScratch(const aixb200_tensor* a, const aixb200_tensor* r);
    void argmax(const aixb200_tensor* a, const aixb200_tensor* r);
    void argmaxIndices(const aixb200_tensor* a, const aixb200_tensor* r);
    void reduceTo(const aixb200_tensor* src, const aixb200_tensor* dst, bool isMax);
    void argmaxTo(const aixb200_tensor* src, const aixb200_tensor* dst, size_t dim, bool oneHot);
    void matmul(const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r);
    void transpose(const aixb200_tensor* a, const aixb200_tensor* r, size_t dim0, size_t dim1);
    void copy(const void* src, uint32_t srcDtype, void* dst, uint32_t dstDtype, size_t count, bool immediate);
    void contiguous(const aixb200_tensor* src, const aixb200_tensor* dst);
    void sliceSet(const aixb200_tensor* src, const aixb200_tensor* dst, size_t dim, size_t start, size_t end, size_t step);
    void triangle(const aixb200_tensor* src, const aixb200_tensor* dst, int64_t diagonal, bool lower);
    void indexSelect(const aixb200_tensor* src, const aixb200_tensor* dst, const aixb200_tensor* idx, size_t dim);
    void indexAdd(const aixb200_tensor* src, const aixb200_tensor* dst, const aixb200_tensor* idx, size_t dim);

    // timing / diagnostics
    void flushL2();
    void selfTestBoundedWait(uint64_t limitNs);
    void fillStats(aixb200_stats* out) const;
    const char* lastKernelSource() const { return m_lastSource.empty() ? nullptr : m_lastSource.c_str(); }

    // data-parallel exchange
    void commInit(int rank, int nranks, const void* id);
    void allReduce(void* data, size_t count, uint32_t dtype, double scale);
    void allReduceAsync(void* data, size_t count, uint32_t dtype, double scale);
    void reduceScatterAsync(void* data, size_t count, uint32_t dtype, double scale);
    void allGatherAsync(void* data, size_t count, uint32_t dtype);
    int  commRank() const;
    int  commSize() const;
    void commWait();
    void commWaitFor(const void* data, size_t bytes);
    void commDestroy();

    // Scratch for fixed kernels (reduction partials, counters); lives as long as the device.
    void* scratch() const { return m_scratch; }
    uint32_t* gemmLaunchCounter() { return &m_gemmLaunches; }
    size_t scratchBytes() const { return m_scratchBytes; }

    std::string lastError;

    // A view whose data is guaranteed to be readable by kernels on the stream. Host memory is staged.
    View inputView(const aixb200_tensor* t, const char* what);
    // A view that kernels may write: memory from this device's allocator (or foreign *device* memory).
    View outputView(const aixb200_tensor* t, const char* what);
    void countLaunch(bool generated) { ++m_stats.total_kernel_launches; if (!generated) ++m_stats.static_kernel_launches; }
    void checkLaunch(const char* what);
    // Temporary device block that is returned to the cache after the next flush.
    void* temporary(size_t bytes);

    // ---- prepared f32 matmul operands ----------------------------------------------------------------------------------
    // The tensor-core f32 product reads every operand as two scaled fp16 terms (gemm_sm100.cu). A tensor is prepared once,
    // in its own row-major layout [rows][2 * paddedCols] = [h0 | h1] per row, and that form serves every orientation the
    // tensor is used in (forward, dX and dW read the same activations, weights and gradients); it is kept until any op
    // writes into the tensor's bytes, the tensor is deallocated, or the cache outgrows its budget.
    struct PreparedTerms
    {
        const char* lo; const char* hi;     // bytes of the source tensor
        uint64_t rows, cols, pitch;         // source layout: rows x cols f32, `pitch` elements between rows
        uint64_t paddedCols;                // multiple of 128
        uint64_t termPitch;                 // fp16 elements between rows of `terms`: 2 * paddedCols plus an optional pad
        void*    terms;                     // device block of rows * 2 * paddedCols fp16
        uint32_t slot;                      // index of the bit pattern of max|x| in the slot block
        bool     ownsSlot;                  // false: the slot belongs to the operand's region (its producer left the maximum there)
        size_t   bytes;
        uint64_t stamp;
    };
    // Returns the cached form or nullptr; `fresh` receives a new entry (terms allocated, not yet filled) when absent.
    const PreparedTerms* findPreparedTerms(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch);
    const PreparedTerms* addPreparedTerms(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch);
    uint32_t* preparedSlot(uint32_t slot) const { return static_cast<uint32_t*>(m_termSlots) + slot; }
    void invalidatePreparedTerms(const void* lo, const void* hi, bool freed = false);
    bool preparedTermsEnabled() const { return m_termCacheEnabled; }
    // max|x| of a matmul operand, left by the kernel that produced it. Tensors that were f32 matmul operands are remembered
    // by address range; when a generated kernel stores exactly such a range, it folds max|x| of what it stores as one more
    // reduction epilogue into the range's slot, and the next preparation of that operand skips its max pass. Returns the
    // slot index, or -1 when no fresh maximum is known.
    int freshOperandMax(const void* lo, const void* hi) const;
    bool ownsMemory(const void* p) const { return m_allocator->findBlock(p) != nullptr; }
    // Called at the top of every C-ABI entry: the host operands the previous call staged are consumed by work that is
    // recorded or enqueued by now, so their blocks may follow the usual deferred-release path.
    void beginCall() { if (!m_staged.empty()) retireStaged(); m_callRanges.clear(); }
    // Byte range the call in progress reads or writes outside the recorder's view (immediate kernels, copies, collectives).
    void noteCallRange(const void* lo, const void* hi) { m_callRanges.push_back({static_cast<const char*>(lo), static_cast<const char*>(hi)}); }

private:
    void record(OpRecord&& rec);
    // ---- matmul with folded consumers ----------------------------------------------------------------------------------
    // nn::Linear is matmul(x, W) + b, usually followed by tanh (aixNeuralNetwork.hpp:150-153). An f32 product the tensor-core
    // kernel can fold consumers into is therefore not launched by the matmul call itself: it waits for the recorded ops
    // that follow. If the first op that touches its result is `result + row vector`, that add is a candidate for the
    // product's epilogue; if the first op that touches the sum is its tanh, that one too. When the wait ends - the tanh
    // has arrived, some other op touches the sum, or anything flushes - the consumers are folded as far as the values they
    // consume are dead (temporaries already deallocated, read by nothing else): the kernel then writes only the sum, or
    // only its tanh, and the folded ops are dropped from the record. Values that stay alive (autograd keeps the product and
    // the sum of every layer) are written by the kernels that always wrote them: see launchDeferredMatmul for the
    // measurement behind that rule. The product is always launched ahead of the ops recorded after it.
    struct DeferredMatmul
    {
        bool active = false;
        aixb200_tensor a{}, b{}, r{};
        View va, vb, vr;
        int folded = 0;                         // recorded consumers matched so far: 0, 1 (the add), 2 (add and tanh)
        size_t addIndex = 0, tanhIndex = 0;     // their positions in m_pending
        View bias, biasOut, tanhOut;
        // Accumulation into a buffer whose zero-fill is still recorded (`grad += dW` after zeroGrad()): the product can be
        // written straight into that buffer, and the fill and the add dropped, if the product itself is dead by then.
        bool   redirect = false;
        size_t fillIndex = 0;                   // position of the zero-fill in m_pending; the add sits at addIndex, its result in biasOut
    };
    DeferredMatmul m_deferred;
    bool m_foldMatmulEpilogue = true;           // AIXB200_GEMM_EPILOGUE=0: every product is launched by its own call
    int  m_foldDepth = 1;                       // consumers folded at most: 1 = the add, 2 = the add and its tanh (AIXB200_GEMM_EPILOGUE=2)
    void advanceDeferredMatmul(size_t index);   // looks at the op just recorded at m_pending[index]
    void launchDeferredMatmul(bool consumerRecorded = false);   // consumerRecorded: a recorded op that reads the sum ended the wait
    void launchMatmul(const DeferredMatmul& d, int folded, void* redirectTo = nullptr);
    bool m_redirectMatmul = true;               // AIXB200_GEMM_REDIRECT=0: accumulations into zero-filled buffers stay kernels of their own
    void launchSpec(const KernelSpec& spec);
    CompiledKernel& getKernel(const KernelSpec& spec, const KernelVariant& variant, const std::string& key);
    std::vector<char> compile(const std::string& source, const std::string& entry);
    bool isHostPointer(const void* p) const;
    void releaseDeferred();
    void retireStaged();

    aixb200_config m_cfg;
    std::string    m_name;
    cudaStream_t   m_stream = nullptr;
    bool           m_ownStream = false;
    int            m_smCount = 148;
    uint64_t       m_totalMemory = 0;
    std::unique_ptr<CachingAllocator> m_allocator;
    void*          m_scratch = nullptr;
    size_t         m_scratchBytes = 0;
    void*          m_l2Flush = nullptr;
    size_t         m_l2FlushBytes = 0;

    std::vector<OpRecord> m_pending;
    std::unordered_set<const void*> m_released;        // storages deallocated while ops were pending
    std::vector<void*> m_deferredFrees;
    std::vector<void*> m_staged;                       // staging copies of host operands of the call in progress
    std::vector<std::pair<const char*, const char*>> m_callRanges;
    bool m_keepIdleFills = true;                       // AIXB200_KEEP_IDLE_FILLS=0: every flush emits every recorded fill
    uint64_t m_deferredBytes = 0;
    PlannerLimits  m_limits;
    CodegenOptions m_codegen;
    int            m_wavesPerSm = 8;
    bool           m_fuseReductions = true;     // AIXB200_FUSE_REDUCTIONS=0 keeps full reductions as kernels of their own
    bool           m_fuseRowReductions = true;  // AIXB200_FUSE_ROW_REDUCTIONS=0 does the same for reduceTo / maxTo over rows

    std::unordered_map<std::string, CompiledKernel> m_kernels;
    std::string m_cacheDir;
    std::string m_lastSource;
    aixb200_stats m_stats{};
    std::unique_ptr<Comm> m_comm;
    cudaStream_t   m_commStream = nullptr;      // side stream of overlapped all-reduces
    cudaStream_t   m_gatherStream = nullptr;    // second side stream: all-gathers on the communicator's gather lane (comm.hpp)
    cudaEvent_t    m_commFork = nullptr;
    struct CommInFlight { const char* begin; const char* end; cudaEvent_t done; };
    std::vector<CommInFlight> m_commInFlight;   // collectives started on the side stream and not yet joined
    std::vector<cudaEvent_t>  m_commEventPool;
    void orderAfterCollectives(const View& v);
    void startCollective(void* data, size_t count, uint32_t dtype, const char* what, const std::function<void(cudaStream_t)>& issue, bool gatherLane = false);
    void scaleOnCommStream(void* data, size_t count, uint32_t dtype, double scale);  // the device's stream waits for in-flight collectives that touch the view
    struct OperandRegion { const char* lo; const char* hi; uint32_t slot; bool fresh; uint64_t stamp; bool operand; };   // operand: the tensor living there has been a matmul operand
    std::vector<OperandRegion> m_operandRegions;
    std::vector<size_t> m_operandSizes;     // byte sizes of tensors that have been f32 matmul operands
    uint32_t m_dummySlot = 0;               // where an epilogue writes when no region could be had
    int  rememberOperandRegion(const char* lo, const char* hi, bool operandNow);
    void appendOperandMaxEpilogues(std::vector<KernelSpec>& kernels, std::vector<std::vector<std::pair<const char*, const char*>>>& regionsOf);
    bool m_fuseOperandMax = true;           // AIXB200_FUSE_OPERAND_MAX=0: every preparation runs its own max pass
    std::vector<PreparedTerms> m_preparedTerms;
    std::vector<uint32_t> m_freeTermSlots;
    void*    m_termSlots = nullptr;
    uint64_t m_preparedBytes = 0, m_preparedStamp = 0;
    bool     m_termCacheEnabled = true;     // AIXB200_GEMM_TERM_CACHE=0: every matmul prepares its operands afresh
    bool m_inFlush = false;
    int  m_residentGrid = 2;                // generated kernels get SMs x resident CTAs x this many CTAs; 0: always SMs x 8 (AIXB200_RESIDENT_GRID)
    uint32_t m_gemmLaunches = 0;            // numbers the launches that use the matmul's tile scheduler in this device's scratch
    bool m_checkErrorWord = false;
};

}   // namespace aixb200
