#include "device.hpp"

#include "comm.hpp"
#include "gemm.hpp"
#include "kernels.hpp"

#include <cuda.h>
#include <cuda_runtime.h>
#include <nvrtc.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sys/stat.h>
#include <unistd.h>

namespace aixb200
{

namespace
{

void check(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) failRuntime(std::string(what) + ": " + cudaGetErrorString(e));
}

// The few driver-API entry points the device needs, fetched through the runtime so that the library does not link
// against libcuda (it must load on machines without a driver).
struct DriverApi
{
    CUresult (*moduleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*moduleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*moduleUnload)(CUmodule) = nullptr;
    CUresult (*launchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*getErrorString)(CUresult, const char**) = nullptr;
    CUresult (*occupancyMaxActiveBlocks)(int*, CUfunction, int, size_t) = nullptr;
    bool loaded = false;
};

DriverApi& driver()
{
    static DriverApi api;
    if (!api.loaded)
    {
        auto get = [](const char* name, void** fn)
        {
            cudaDriverEntryPointQueryResult status;
            check(cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &status), name);
            if (status != cudaDriverEntryPointSuccess || !*fn) failRuntime(std::string("driver entry point not found: ") + name);
        };
        get("cuModuleLoadData", reinterpret_cast<void**>(&api.moduleLoadData));
        get("cuModuleGetFunction", reinterpret_cast<void**>(&api.moduleGetFunction));
        get("cuModuleUnload", reinterpret_cast<void**>(&api.moduleUnload));
        get("cuLaunchKernel", reinterpret_cast<void**>(&api.launchKernel));
        get("cuGetErrorString", reinterpret_cast<void**>(&api.getErrorString));
        get("cuOccupancyMaxActiveBlocksPerMultiprocessor", reinterpret_cast<void**>(&api.occupancyMaxActiveBlocks));
        api.loaded = true;
    }
    return api;
}

void checkDriver(CUresult r, const char* what)
{
    if (r == CUDA_SUCCESS) return;
    const char* msg = nullptr;
    driver().getErrorString(r, &msg);
    failRuntime(std::string(what) + ": " + (msg ? msg : "unknown driver error"));
}

int envInt(const char* name, int fallback)
{
    const char* v = std::getenv(name);
    return (v && *v) ? std::atoi(v) : fallback;
}

std::string hex64(uint64_t v)
{
    char buf[17];
    std::snprintf(buf, sizeof(buf), "%016llx", static_cast<unsigned long long>(v));
    return buf;
}

}   // namespace

// ----------------------------------------------------------------------------------------------------------------
// construction / destruction
// ----------------------------------------------------------------------------------------------------------------
Device::Device(const aixb200_config& cfg) : m_cfg(cfg)
{
    if (m_cfg.flush_threshold == 0) m_cfg.flush_threshold = 200;
    m_limits.fusion = m_cfg.fusion != 0;
    m_codegen.strictMath = m_cfg.strict_math != 0;
    m_codegen.block = envInt("AIXB200_EW_BLOCK", 256);
    m_codegen.unroll = std::max(1, std::min(8, envInt("AIXB200_EW_UNROLL", 2)));
    m_codegen.rowMinBlocks = std::max(-1, std::min(8, envInt("AIXB200_ROW_MIN_BLOCKS", -1)));
    m_wavesPerSm = std::max(1, envInt("AIXB200_EW_WAVES", 8));
    m_fuseReductions = envInt("AIXB200_FUSE_REDUCTIONS", 1) != 0;
    m_fuseRowReductions = envInt("AIXB200_FUSE_ROW_REDUCTIONS", 1) != 0;
    m_termCacheEnabled = envInt("AIXB200_GEMM_TERM_CACHE", 1) != 0;
    m_keepIdleFills = envInt("AIXB200_KEEP_IDLE_FILLS", 1) != 0;
    m_fuseOperandMax = envInt("AIXB200_FUSE_OPERAND_MAX", 1) != 0;
    // 0: every product is launched by its own call; 1 (default): `+ row vector` may be folded; 2: its tanh as well (measured
    // slower than the separate kernel: see launchDeferredMatmul)
    m_foldDepth = std::max(0, std::min(2, envInt("AIXB200_GEMM_EPILOGUE", 1)));
    m_foldMatmulEpilogue = m_foldDepth != 0 && m_cfg.strict_math == 0 && m_cfg.fusion != 0;
    m_redirectMatmul = envInt("AIXB200_GEMM_REDIRECT", 1) != 0;
    m_residentGrid = std::max(0, std::min(4, envInt("AIXB200_RESIDENT_GRID", 2)));

    if (m_cfg.disk_cache)
    {
        const char* dir = std::getenv("AIXB200_CACHE_DIR");
        if (dir && *dir) m_cacheDir = dir;
        else
        {
            const char* home = std::getenv("HOME");
            m_cacheDir = std::string(home && *home ? home : "/tmp") + "/.cache/aixb200";
        }
        ::mkdir((m_cacheDir.substr(0, m_cacheDir.find_last_of('/'))).c_str(), 0755);
        ::mkdir(m_cacheDir.c_str(), 0755);
    }

    if (dryRun())
    {
        m_name = "B200 (dry run, no GPU)";
        RawMemoryOps raw;
        const uint64_t injected = m_cfg.inject_alloc_limit_bytes;
        raw.allocate = [injected, this](size_t bytes) -> void*
        {
            if (injected && m_allocator && m_allocator->bytesReserved() + bytes > injected) return nullptr;     // injected out-of-memory
            return std::malloc(bytes);
        };
        raw.free = [](void* p) { std::free(p); };
        m_allocator = std::make_unique<CachingAllocator>(raw, uint64_t(1) << 30);
        return;
    }

    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
        throw Error(AIXB200_ERR_NOGPU, "no CUDA device is visible; the B200 device has no CPU fallback");
    if (m_cfg.ordinal < 0 || m_cfg.ordinal >= count) failInvalid("device ordinal out of range");
    check(cudaSetDevice(m_cfg.ordinal), "cudaSetDevice");
    cudaDeviceProp prop{};
    check(cudaGetDeviceProperties(&prop, m_cfg.ordinal), "cudaGetDeviceProperties");
    if (prop.major != 10)
        throw Error(AIXB200_ERR_NOGPU, std::string("device '") + prop.name + "' is not sm_100 (Blackwell B200); kernels are built for sm_100a only");
    m_name = std::string("B200:") + prop.name;
    m_smCount = prop.multiProcessorCount;
    m_totalMemory = prop.totalGlobalMem;
    driver();

    if (m_cfg.stream) m_stream = static_cast<cudaStream_t>(m_cfg.stream);
    else
    {
        check(cudaStreamCreateWithFlags(&m_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        m_ownStream = true;
    }

    const bool managed = m_cfg.managed_memory != 0;
    const int ordinal = m_cfg.ordinal;
    RawMemoryOps raw;
    const uint64_t injected = m_cfg.inject_alloc_limit_bytes;
    raw.allocate = [managed, ordinal, injected, this](size_t bytes) -> void*
    {
        if (injected && m_allocator && m_allocator->bytesReserved() + bytes > injected) return nullptr;         // injected out-of-memory
        void* p = nullptr;
        cudaError_t e = managed ? cudaMallocManaged(&p, bytes) : cudaMalloc(&p, bytes);
        if (e == cudaErrorMemoryAllocation) { cudaGetLastError(); return nullptr; }
        check(e, "cudaMalloc");
        if (managed)
        {
            // Keep the pages on the GPU; the host reads them after synchronize() through on-demand migration.
            cudaMemLocation loc{};
            loc.type = cudaMemLocationTypeDevice;
            loc.id = ordinal;
            cudaMemAdvise_v2(p, bytes, cudaMemAdviseSetPreferredLocation, loc);
            cudaMemPrefetchAsync_v2(p, bytes, loc, 0, m_stream);
            cudaGetLastError();
        }
        ++m_stats.cuda_mallocs;
        return p;
    };
    raw.free = [](void* p) { cudaFree(p); };
    uint64_t limit = m_cfg.cache_limit_bytes ? m_cfg.cache_limit_bytes : m_totalMemory / 4 * 3;
    m_allocator = std::make_unique<CachingAllocator>(raw, limit);

    m_scratchBytes = size_t(4) << 20;
    check(cudaMalloc(&m_scratch, m_scratchBytes + kernels::kGemmCounterBytes), "cudaMalloc(scratch)");
    check(cudaMemsetAsync(m_scratch, 0, m_scratchBytes + kernels::kGemmCounterBytes, m_stream), "cudaMemset(scratch)");
}

Device::~Device()
{
    if (!dryRun())
    {
        cudaSetDevice(m_cfg.ordinal);
        if (m_commStream) cudaStreamSynchronize(m_commStream);
        if (m_gatherStream) cudaStreamSynchronize(m_gatherStream);
        m_comm.reset();
        if (m_gatherStream) { cudaStreamDestroy(m_gatherStream); m_gatherStream = nullptr; }
        if (m_commStream)
        {
            cudaStreamDestroy(m_commStream); cudaEventDestroy(m_commFork);
            for (const CommInFlight& c : m_commInFlight) cudaEventDestroy(c.done);
            for (cudaEvent_t e : m_commEventPool) cudaEventDestroy(e);
        }
        if (m_stream) cudaStreamSynchronize(m_stream);
        for (auto& [key, k] : m_kernels)
            if (k.module) driver().moduleUnload(k.module);
        if (m_scratch) cudaFree(m_scratch);
        if (m_l2Flush) cudaFree(m_l2Flush);
    }
    m_allocator.reset();
    if (!dryRun() && m_ownStream && m_stream) cudaStreamDestroy(m_stream);
}

// ----------------------------------------------------------------------------------------------------------------
// memory
// ----------------------------------------------------------------------------------------------------------------
void* Device::allocate(size_t bytes)
{
    // Headroom of one 16-byte pack so that vector tails stay inside the block (the reference pads to 4 elements,
    // aixDeviceMetal.cpp:245-248).
    try
    {
        return m_allocator->allocate(bytes + 16);
    }
    catch (const Error&)
    {
        // Out of memory with dead buffers still parked behind recorded ops: emit those ops (which returns the buffers
        // to the cache), then try once more.
        if (m_deferredFrees.empty() || m_inFlush) throw;
        flushAll();
        return m_allocator->allocate(bytes + 16);
    }
}

void* Device::temporary(size_t bytes)
{
    void* p = m_allocator->allocate(bytes + 16);
    m_released.insert(p);
    m_deferredFrees.push_back(p);
    m_deferredBytes += m_allocator->blockSize(p);
    return p;
}

// ---- prepared f32 matmul operands (see device.hpp) --------------------------------------------------------------------
const Device::PreparedTerms* Device::findPreparedTerms(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch)
{
    for (PreparedTerms& e : m_preparedTerms)
        if (e.lo == base && e.rows == rows && e.cols == cols && e.pitch == pitch) { e.stamp = ++m_preparedStamp; ++m_stats.prepared_operand_hits; return &e; }
    return nullptr;
}

const Device::PreparedTerms* Device::addPreparedTerms(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch)
{
    constexpr uint32_t kSlots = 1024;
    if (!m_termSlots)
    {
        m_termSlots = m_allocator->allocate(kSlots * sizeof(uint32_t));
        for (uint32_t i = kSlots; i-- > 1;) m_freeTermSlots.push_back(i);
        m_dummySlot = 0;
    }
    PreparedTerms e{};
    e.lo = static_cast<const char*>(base);
    e.hi = e.lo + ((rows - 1) * pitch + cols) * sizeof(float);
    e.rows = rows; e.cols = cols; e.pitch = pitch;
    e.paddedCols = (cols + 127) & ~uint64_t(127);
    // AIXB200_GEMM_TERM_PAD: extra fp16 elements per row (a multiple of 8), so that rows do not sit a power of two apart
    static const uint64_t pad = []{ const char* v = std::getenv("AIXB200_GEMM_TERM_PAD"); return v ? (std::strtoull(v, nullptr, 10) & ~uint64_t(7)) : uint64_t(0); }();
    e.termPitch = 2 * e.paddedCols + pad;
    e.bytes = static_cast<size_t>(rows) * e.termPitch * sizeof(uint16_t);
    // budget: an eighth of the device memory, oldest entries go first
    const uint64_t budget = std::max<uint64_t>(m_totalMemory / 8, e.bytes);
    while (!m_preparedTerms.empty() && (m_preparedBytes + e.bytes > budget || m_freeTermSlots.empty()))
    {
        size_t oldest = 0;
        for (size_t i = 1; i < m_preparedTerms.size(); ++i)
            if (m_preparedTerms[i].stamp < m_preparedTerms[oldest].stamp) oldest = i;
        const PreparedTerms victim = m_preparedTerms[oldest];
        if (victim.stamp == m_preparedStamp) break;         // the other operand of the matmul being launched: never evicted
        invalidatePreparedTerms(victim.lo, victim.hi);
    }
    e.terms = m_allocator->allocate(e.bytes + 16);
    const int produced = freshOperandMax(e.lo, e.hi);
    if (produced >= 0) { e.slot = static_cast<uint32_t>(produced); e.ownsSlot = false; ++m_stats.prepared_operand_max_known; }
    else
    {
        e.slot = m_freeTermSlots.back();
        m_freeTermSlots.pop_back();
        e.ownsSlot = true;
    }
    rememberOperandRegion(e.lo, e.hi, true);
    e.stamp = ++m_preparedStamp;
    m_preparedBytes += e.bytes;
    ++m_stats.prepared_operand_builds;
    m_preparedTerms.push_back(e);
    return &m_preparedTerms.back();
}

// Every kernel that read a prepared form is already enqueued when this runs (matmuls launch at call time), so the block
// can go back to the allocator at once: reuse is ordered behind those kernels on the device's stream.
int Device::freshOperandMax(const void* lo, const void* hi) const
{
    for (const OperandRegion& r : m_operandRegions)
        if (r.lo == lo && r.hi == hi) return r.fresh ? static_cast<int>(r.slot) : -1;
    return -1;
}

// Returns the index of the range's entry (created if need be), or -1. `operandNow`: the range is being prepared as a matmul
// operand - its size joins the sizes whose producers are asked for max|x|.
int Device::rememberOperandRegion(const char* lo, const char* hi, bool operandNow)
{
    const size_t bytes = static_cast<size_t>(hi - lo);
    if (!m_fuseOperandMax || bytes < (size_t(1) << 20)) return -1;          // small operands: the max pass is noise
    if (operandNow && std::find(m_operandSizes.begin(), m_operandSizes.end(), bytes) == m_operandSizes.end() && m_operandSizes.size() < 32)
        m_operandSizes.push_back(bytes);
    for (size_t i = 0; i < m_operandRegions.size(); ++i)
        if (m_operandRegions[i].lo == lo && m_operandRegions[i].hi == hi)
        {
            m_operandRegions[i].stamp = ++m_preparedStamp;
            m_operandRegions[i].operand = m_operandRegions[i].operand || operandNow;
            return static_cast<int>(i);
        }
    if (m_operandRegions.size() >= 64 || m_freeTermSlots.size() < 64)
    {
        // forget the range used longest ago, unless a prepared form still reads its slot
        size_t oldest = m_operandRegions.size();
        for (size_t i = 0; i < m_operandRegions.size(); ++i)
        {
            bool inUse = false;
            for (const PreparedTerms& e : m_preparedTerms) inUse = inUse || (!e.ownsSlot && e.slot == m_operandRegions[i].slot);
            if (!inUse && (oldest == m_operandRegions.size() || m_operandRegions[i].stamp < m_operandRegions[oldest].stamp)) oldest = i;
        }
        if (oldest == m_operandRegions.size()) return -1;
        m_freeTermSlots.push_back(m_operandRegions[oldest].slot);
        m_operandRegions[oldest] = m_operandRegions.back();
        m_operandRegions.pop_back();
    }
    if (m_freeTermSlots.empty()) return -1;
    m_operandRegions.push_back({lo, hi, m_freeTermSlots.back(), false, ++m_preparedStamp, operandNow});
    m_freeTermSlots.pop_back();
    return static_cast<int>(m_operandRegions.size() - 1);
}

// A generated kernel folds max|x| of a dense f32 tensor it stores into that tensor's slot when the tensor has the size of
// earlier matmul operands and either is the kernel's only such store (activations, gradients: fresh allocations whose
// addresses vary - the choice then depends on sizes only, so the kernel's identity is stable) or lives where a matmul operand
// lives (weights updated in place next to optimizer state of the same size). regionsOf[k] lists the ranges kernel k refreshes.
void Device::appendOperandMaxEpilogues(std::vector<KernelSpec>& kernels, std::vector<std::vector<std::pair<const char*, const char*>>>& regionsOf)
{
    regionsOf.assign(kernels.size(), {});
    if (m_operandSizes.empty() || !m_fuseReductions || !m_termSlots) return;
    for (size_t k = 0; k < kernels.size(); ++k)
    {
        KernelSpec& spec = kernels[k];
        auto qualifies = [&](const KernelStore& st)
        {
            if (st.view.dtype != F32 || !st.view.isDense() || st.view.size != spec.count) return false;
            const size_t bytes = static_cast<size_t>(st.view.endByte() - st.view.firstByte());
            return std::find(m_operandSizes.begin(), m_operandSizes.end(), bytes) != m_operandSizes.end();
        };
        size_t candidates = 0, known = 0;
        int lastNode = -1;
        auto livesThere = [&](const KernelStore& st)
        {
            for (const OperandRegion& r : m_operandRegions)
                if (r.operand && r.lo == st.view.firstByte() && r.hi == st.view.endByte()) return true;
            return false;
        };
        for (const KernelStore& st : spec.stores)
            if (qualifies(st)) { ++candidates; known += livesThere(st) ? 1 : 0; lastNode = std::max(lastNode, static_cast<int>(st.node)); }
        for (const KernelStore& st : spec.stores)
        {
            if (!qualifies(st)) continue;
            if (spec.reductions.size() >= m_limits.maxReductionsPerKernel) break;
            // Several candidates: those where an operand is known to live; if none is, the value computed last - the end of
            // the chain is what the next matmul reads (bias + tanh stores the sum and its tanh; the tanh is the operand).
            // Both choices depend on the recorded ops and on sizes only, not on the addresses of fresh allocations.
            if (candidates > 1 && (known > 0 ? !livesThere(st) : static_cast<int>(st.node) != lastNode)) continue;
            const int region = rememberOperandRegion(st.view.firstByte(), st.view.endByte(), false);
            View slot;
            slot.base = reinterpret_cast<char*>(preparedSlot(region >= 0 ? m_operandRegions[static_cast<size_t>(region)].slot : m_dummySlot));
            slot.size = 1;
            slot.dtype = F32;
            spec.reductions.push_back({st.node, true, static_cast<uint8_t>(F32), slot, true});
            if (region >= 0) regionsOf[k].push_back({st.view.firstByte(), st.view.endByte()});
        }
    }
}

void Device::invalidatePreparedTerms(const void* lo, const void* hi, bool freed)
{
    {
        // whatever is written into an operand's range, the maximum its producer left is stale; once the memory is freed,
        // whatever lives there next is not the operand any more
        const char* first = static_cast<const char*>(lo);
        const char* last = static_cast<const char*>(hi);
        for (OperandRegion& r : m_operandRegions)
            if (first < r.hi && r.lo < last) { r.fresh = false; if (freed) r.operand = false; }
    }
    if (m_preparedTerms.empty()) return;
    const char* first = static_cast<const char*>(lo);
    const char* last = static_cast<const char*>(hi);
    for (size_t i = 0; i < m_preparedTerms.size();)
    {
        PreparedTerms& e = m_preparedTerms[i];
        if (first < e.hi && e.lo < last)
        {
            m_allocator->release(e.terms);
            if (e.ownsSlot) m_freeTermSlots.push_back(e.slot);
            m_preparedBytes -= e.bytes;
            m_preparedTerms[i] = m_preparedTerms.back();
            m_preparedTerms.pop_back();
        }
        else ++i;
    }
}

// Staged host operands stay out of the deferred-release list while the call that staged them is still running: a flush
// inside that call (ordering after a collective, the flush every immediate op starts with) returns deferred blocks to
// the cache, and the call's own temporaries could then be handed the very block its operand sits in.
void Device::retireStaged()
{
    for (void* p : m_staged)
    {
        invalidatePreparedTerms(p, static_cast<char*>(p) + m_allocator->blockSize(p), true);     // the block will hold other data next
        m_released.insert(p);
        m_deferredFrees.push_back(p);
        m_deferredBytes += m_allocator->blockSize(p);
    }
    m_staged.clear();
}

void Device::deallocate(void* p)
{
    if (!p) return;
    if (!m_allocator->owns(p)) failInvalid("deallocate: pointer was not allocated by this device");
    if (m_released.count(p)) failInvalid("deallocate: pointer was already deallocated");
    invalidatePreparedTerms(p, static_cast<char*>(p) + m_allocator->blockSize(p), true);
    if (!m_commInFlight.empty())
    {
        // a collective on the side stream may still use the block: reuse is ordered on the device's stream only
        aixb200_tensor whole{};
        whole.data = p; whole.size = m_allocator->blockSize(p); whole.dtype = U8; whole.rank = 1; whole.shape[0] = whole.size; whole.strides[0] = 1;
        noteCallRange(p, static_cast<char*>(p) + whole.size);
        orderAfterCollectives(makeView(&whole, "deallocate"));
    }
    if (m_pending.empty() && m_deferredFrees.empty() && !m_deferred.active)
    {
        m_allocator->release(p);       // stream order makes immediate reuse safe
        return;
    }
    m_released.insert(p);
    m_deferredFrees.push_back(p);
    m_deferredBytes += m_allocator->blockSize(p);
    // Memory pressure: do not let dead buffers pile up behind a long recorded chain
    // (the reference commits when half its working-set budget is queued, aixDeviceMetal.cpp:1438-1444).
    const uint64_t budget = dryRun() ? (uint64_t(1) << 30) : m_totalMemory / 2;
    if (m_deferredBytes > budget) flushAll();
}

void Device::releaseDeferred()
{
    for (void* p : m_deferredFrees) m_allocator->release(p);
    m_deferredFrees.clear();
    m_released.clear();
    m_deferredBytes = 0;
}

void Device::emptyCache()
{
    flushAll();
    if (!dryRun()) check(cudaStreamSynchronize(m_stream), "synchronize");
    invalidatePreparedTerms(nullptr, reinterpret_cast<const void*>(~uintptr_t(0)));
    m_allocator->trim(0);
}

void Device::synchronize()
{
    flushAll();
    if (dryRun()) { if (m_comm && !m_comm->aborted()) m_comm->checkAsyncError("synchronize"); return; }
    // With managed memory the host may write into any tensor through its pointer once the device is idle: nothing
    // prepared from the tensors' contents survives a synchronisation.
    if (m_cfg.managed_memory) invalidatePreparedTerms(nullptr, reinterpret_cast<const void*>(~uintptr_t(0)));
    commWait();
    check(cudaStreamSynchronize(m_stream), "cudaStreamSynchronize");
    check(cudaGetLastError(), "asynchronous kernel failure");
    if (m_checkErrorWord)
    {
        // Kernels never trap: one with a bounded wait (tensor-core GEMM) that ran out, or one that met an index outside
        // its dimension, raises a word in scratch, skips the work it cannot do, and the failure surfaces here.
        m_checkErrorWord = false;
        uint32_t words[2] = {0, 0};
        check(cudaMemcpy(words, static_cast<char*>(m_scratch) + kernels::kScratchTimeoutOffset, 8, cudaMemcpyDeviceToHost), "read error words");
        if (words[0] || words[1])
        {
            cudaMemset(static_cast<char*>(m_scratch) + kernels::kScratchTimeoutOffset, 0, 8);
            if (words[0])
            {
                cudaMemset(static_cast<char*>(m_scratch) + m_scratchBytes, 0, kernels::kGemmCounterBytes);   // split-tile counters
                throw Error(AIXB200_ERR_TIMEOUT, "a bounded device-side wait ran out; the result of the kernel that waited is invalid");
            }
            throw Error(AIXB200_ERR_INVALID, "indexSelect / indexAdd: an index lies outside the indexed dimension; those elements were skipped");
        }
    }
}

bool Device::isHostPointer(const void* p) const
{
    if (dryRun()) return false;
    cudaPointerAttributes attr{};
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) { cudaGetLastError(); return true; }
    return attr.type == cudaMemoryTypeUnregistered || attr.type == cudaMemoryTypeHost;
}

View Device::inputView(const aixb200_tensor* t, const char* what)
{
    View v = makeView(t, what);
    if (v.size != 0) noteCallRange(v.firstByte(), v.endByte());
    if (v.size == 0 || dryRun()) return v;
    if (!m_commInFlight.empty()) orderAfterCollectives(v);
    if (m_allocator->findBlock(v.base)) return v;
    if (!isHostPointer(v.base)) return v;                 // foreign device memory (another allocator in this process)
    // Host memory (the reference's getReadOnlyMTLBuffer path, aixDeviceMetal.cpp:1478-1490): copy the touched span
    // to a temporary device block now; program order on the stream keeps it ahead of the kernels that read it.
    const size_t es = dtypeSize(v.dtype);
    const size_t bytes = v.span() * es;
    char* staged = static_cast<char*>(m_allocator->allocate(bytes + 16));
    m_staged.push_back(staged);
    check(cudaMemcpyAsync(staged, v.firstByte(), bytes, cudaMemcpyHostToDevice, m_stream), "host-to-device staging copy");
    m_stats.h2d_bytes += bytes;
    v.base = staged;
    v.offset = 0;
    return v;
}

View Device::outputView(const aixb200_tensor* t, const char* what)
{
    View v = makeView(t, what);
    if (v.size != 0) noteCallRange(v.firstByte(), v.endByte());
    if (v.size == 0 || dryRun()) return v;
    invalidatePreparedTerms(v.firstByte(), v.endByte());       // whatever is written here, its prepared matmul form is stale
    if (!m_commInFlight.empty()) orderAfterCollectives(v);
    if (m_allocator->findBlock(v.base)) return v;
    if (isHostPointer(v.base)) failInvalid(std::string(what) + ": result must be device memory allocated by this device");
    return v;
}

void Device::checkLaunch(const char* what)
{
    if (dryRun()) return;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        // a matmul that was not launched has not prepared its tile scheduler's next counter: start that area afresh
        cudaMemsetAsync(static_cast<char*>(m_scratch) + m_scratchBytes, 0, kernels::kGemmCounterBytes, m_stream);
        failRuntime(std::string(what) + ": " + cudaGetErrorString(e));
    }
}

// ----------------------------------------------------------------------------------------------------------------
// recording
// ----------------------------------------------------------------------------------------------------------------
void Device::record(OpRecord&& rec)
{
    if (rec.out.size == 0) return;
    m_pending.push_back(std::move(rec));
    ++m_stats.ops_recorded;
    if (m_deferred.active) advanceDeferredMatmul(m_pending.size() - 1);
    if (m_pending.size() >= m_cfg.flush_threshold) flush();
}

static void checkOperandSize(const View& in, const View& out, const char* what)
{
    if (in.size != out.size && in.size != 1)
        failInvalid(std::string(what) + ": operand has " + std::to_string(in.size) + " elements, result has " + std::to_string(out.size));
}

void Device::recordBinary(Op op, const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r, const char* what)
{
    OpRecord rec;
    rec.op = op;
    rec.numInputs = 2;
    rec.out = outputView(r, what);
    rec.in[0] = inputView(a, what);
    rec.in[1] = inputView(b, what);
    checkOperandSize(rec.in[0], rec.out, what);
    checkOperandSize(rec.in[1], rec.out, what);
    record(std::move(rec));
}

void Device::recordUnary(Op op, const aixb200_tensor* a, const aixb200_tensor* r, const char* what)
{
    OpRecord rec;
    rec.op = op;
    rec.numInputs = 1;
    rec.out = outputView(r, what);
    rec.in[0] = inputView(a, what);
    checkOperandSize(rec.in[0], rec.out, what);
    record(std::move(rec));
}

void Device::recordFill(const void* scalar, uint32_t scalarDtype, const aixb200_tensor* r)
{
    if (!scalar) failInvalid("fill: null scalar");
    dtypeSize(scalarDtype);
    OpRecord rec;
    rec.op = Op::Fill;
    rec.out = outputView(r, "fill");
    rec.scalar = convertScalar(scalar, scalarDtype, rec.out.dtype);
    record(std::move(rec));
}

void Device::recordFillMin(const aixb200_tensor* r)
{
    OpRecord rec;
    rec.op = Op::Fill;
    rec.out = outputView(r, "fillMin");
    rec.scalar = lowestValue(rec.out.dtype);
    record(std::move(rec));
}

// ----------------------------------------------------------------------------------------------------------------
// flush: plan, generate, compile, launch
// ----------------------------------------------------------------------------------------------------------------
void Device::flush(bool keepIdleFills)
{
    if (m_inFlush) return;
    if (m_deferred.active) launchDeferredMatmul();        // issued before everything recorded after it
    if (m_pending.empty()) { releaseDeferred(); return; }
    m_inFlush = true;
    struct Reset { bool& f; ~Reset() { f = false; } } reset{m_inFlush};
    std::vector<OpRecord> ops;
    ops.swap(m_pending);
    if (keepIdleFills && m_keepIdleFills && m_limits.fusion)
    {
        // Idle fills stay recorded (see the declaration). "Idle": alive storage, untouched by every other op of the batch
        // and by the call in progress.
        auto meet = [](const char* alo, const char* ahi, const char* blo, const char* bhi) { return alo < bhi && blo < ahi; };
        std::vector<char> idle(ops.size(), 0);
        size_t idleCount = 0;
        for (size_t i = 0; i < ops.size(); ++i)
        {
            if (ops[i].op != Op::Fill || m_released.count(ops[i].out.base)) continue;
            const char* lo = ops[i].out.firstByte();
            const char* hi = ops[i].out.endByte();
            bool touched = false;
            for (const auto& r : m_callRanges) touched = touched || meet(lo, hi, r.first, r.second);
            for (size_t j = 0; j < ops.size() && !touched; ++j)
            {
                if (j == i) continue;
                touched = meet(lo, hi, ops[j].out.firstByte(), ops[j].out.endByte());
                for (int k = 0; k < ops[j].numInputs && !touched; ++k) touched = meet(lo, hi, ops[j].in[k].firstByte(), ops[j].in[k].endByte());
            }
            if (!touched) { idle[i] = 1; ++idleCount; }
        }
        if (idleCount > 0 && idleCount <= 64)
        {
            std::vector<OpRecord> rest;
            rest.reserve(ops.size() - idleCount);
            for (size_t i = 0; i < ops.size(); ++i) (idle[i] ? m_pending : rest).push_back(ops[i]);
            ops.swap(rest);
            if (ops.empty()) { releaseDeferred(); return; }
        }
    }
    ++m_stats.flushes;
    try
    {
        std::vector<KernelSpec> kernels = planKernels(ops, m_released, m_limits);
        std::vector<std::vector<std::pair<const char*, const char*>>> refreshed;
        appendOperandMaxEpilogues(kernels, refreshed);
        for (size_t k = 0; k < kernels.size(); ++k)
        {
            const KernelSpec& spec = kernels[k];
            launchSpec(spec);
            for (const auto& range : refreshed[k])
                for (OperandRegion& r : m_operandRegions)
                    if (r.lo == range.first && r.hi == range.second) r.fresh = !dryRun();
            ++m_stats.fused_kernels;
            m_stats.fused_ops += spec.opsFolded;
            m_stats.fills_absorbed += spec.fillsAbsorbed;
            m_stats.stores_elided += spec.storesElided;
        }
    }
    catch (...)
    {
        releaseDeferred();
        throw;
    }
    releaseDeferred();
}

std::vector<char> Device::compile(const std::string& source, const std::string& entry)
{
    std::vector<const char*> options = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device"};
    if (m_codegen.strictMath) { options.push_back("--fmad=false"); options.push_back("--prec-div=true"); options.push_back("--prec-sqrt=true"); }
    else { options.push_back("--fmad=true"); options.push_back("--prec-div=false"); options.push_back("--prec-sqrt=false"); }

    std::string cachePath;
    if (!m_cacheDir.empty())
    {
        uint64_t h = fnv1a(source.data(), source.size());
        for (auto o : options) h = fnv1a(o, std::strlen(o), h);
        cachePath = m_cacheDir + "/" + hex64(h) + ".cubin";
        std::ifstream in(cachePath, std::ios::binary);
        if (in)
        {
            std::vector<char> cubin((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
            if (!cubin.empty()) return cubin;
        }
    }

    if (m_cfg.inject_nvrtc_failures > 0)
    {
        --m_cfg.inject_nvrtc_failures;
        m_lastSource = source;
        failRuntime("NVRTC failed to compile a fused kernel: injected failure (aixb200_config.inject_nvrtc_failures)");
    }
    const auto t0 = std::chrono::steady_clock::now();
    nvrtcProgram prog = nullptr;
    if (nvrtcCreateProgram(&prog, source.c_str(), (entry + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS)
        failRuntime("nvrtcCreateProgram failed");
    nvrtcResult r = nvrtcCompileProgram(prog, static_cast<int>(options.size()), options.data());
    if (r != NVRTC_SUCCESS)
    {
        size_t logSize = 0;
        nvrtcGetProgramLogSize(prog, &logSize);
        std::string log(logSize, '\0');
        if (logSize) nvrtcGetProgramLog(prog, log.data());
        nvrtcDestroyProgram(&prog);
        m_lastSource = source;
        failRuntime("NVRTC failed to compile a fused kernel: " + log);
    }
    size_t size = 0;
    nvrtcGetCUBINSize(prog, &size);
    std::vector<char> cubin(size);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    ++m_stats.nvrtc_compiles;
    m_stats.nvrtc_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();

    if (!cachePath.empty())
    {
        const std::string tmp = cachePath + "." + std::to_string(::getpid());
        std::ofstream out(tmp, std::ios::binary);
        if (out)
        {
            out.write(cubin.data(), static_cast<std::streamsize>(cubin.size()));
            out.close();
            std::rename(tmp.c_str(), cachePath.c_str());
        }
    }
    return cubin;
}

CompiledKernel& Device::getKernel(const KernelSpec& spec, const KernelVariant& variant, const std::string& key)
{
    auto it = m_kernels.find(key);
    if (it != m_kernels.end()) { ++m_stats.kernel_cache_hits; return it->second; }
    ++m_stats.kernel_cache_misses;
    const std::string entry = "aixb200_fused_" + hex64(fnv1a(key.data(), key.size()));
    CompiledKernel k;
    k.source = generateKernelSource(spec, variant, m_codegen, entry);
    std::vector<char> cubin = compile(k.source, entry);
    if (!dryRun())
    {
        checkDriver(driver().moduleLoadData(&k.module, cubin.data()), "cuModuleLoadData");
        checkDriver(driver().moduleGetFunction(&k.function, k.module, entry.c_str()), "cuModuleGetFunction");
        int perSm = 0;
        if (driver().occupancyMaxActiveBlocks(&perSm, k.function, m_codegen.block, 0) == CUDA_SUCCESS && perSm > 0) k.residentPerSm = perSm;
        if (std::getenv("AIXB200_DEBUG_OCCUPANCY")) std::fprintf(stderr, "%s: %d CTAs per SM, %zu nodes\n", entry.c_str(), perSm, spec.nodes.size());
    }
    return m_kernels.emplace(key, std::move(k)).first->second;
}

void Device::launchSpec(const KernelSpec& spec)
{
    const KernelVariant variant = chooseVariant(spec);
    const std::string key = kernelKey(spec, variant, m_codegen);
    CompiledKernel& k = getKernel(spec, variant, key);
    m_lastSource = k.source;
    for (const KernelReduce& r : spec.reductions) m_stats.reductions_fused += r.absBits ? 0 : 1;      // the caller's reductions only
    m_stats.reductions_fused += spec.rowReductions.size();
    if (dryRun()) { countLaunch(true); return; }

    std::vector<uint64_t> args = packKernelArguments(spec, variant, m_scratch);
    if (args.empty()) args.push_back(0);
    const uint64_t block = static_cast<uint64_t>(m_codegen.block);
    const uint64_t nvec = variant.vec > 1 ? spec.count / variant.vec : 0;
    const uint64_t mainBlocks = (nvec + block * m_codegen.unroll - 1) / (block * m_codegen.unroll);
    const uint64_t tailElems = variant.vec > 1 ? spec.count - nvec * variant.vec : spec.count;
    const uint64_t tailBlocks = (tailElems + block - 1) / block;
    uint64_t grid = std::max<uint64_t>(1, std::max(mainBlocks, tailBlocks));
    if (variant.rowMode)
    {
        const uint64_t rows = spec.count / spec.rowCols;
        grid = variant.warpPerRow ? (rows + block / 32 - 1) / (block / 32) : rows;
    }
    // Every generated kernel walks its elements (or rows) with a grid stride, so the grid is free: a whole number of waves of
    // the CTAs that are resident at once. SMs x 8 regardless of occupancy left a partial last wave that ran at a fraction
    // of the bandwidth after everything else had finished; exactly one wave loses the balancing between fast and slow
    // SMs. Measured (chain over 2^28 elements, f32 / bf16, of the copy peak): two waves 0.985 / 0.891, one 0.979 / 0.833,
    // SMs x 8 with five resident 0.971 / 0.880.
    const int perSm = m_residentGrid > 0 && k.residentPerSm > 0 ? std::min(m_wavesPerSm, k.residentPerSm) * m_residentGrid : m_wavesPerSm;
    grid = std::min<uint64_t>(grid, static_cast<uint64_t>(m_smCount) * perSm);
    if (!spec.reductions.empty()) grid = std::min<uint64_t>(grid, kReductionMaxBlocks);    // one scratch partial per block
    void* params[] = {args.data()};
    checkDriver(driver().launchKernel(k.function, static_cast<unsigned>(grid), 1, 1, static_cast<unsigned>(block), 1, 1, 0, m_stream, params, nullptr),
                "cuLaunchKernel(fused)");
    countLaunch(true);
}

// ----------------------------------------------------------------------------------------------------------------
// immediate ops
// ----------------------------------------------------------------------------------------------------------------
namespace
{

kernels::LaunchContext makeContext(Device& d, uint64_t* launches)
{
    return kernels::LaunchContext{d.stream(), d.smCount(), d.scratch(), d.scratchBytes(), launches, d.gemmLaunchCounter()};
}

kernels::Layout layoutOf(const aixb200_tensor* t)
{
    kernels::Layout l{};
    l.rank = static_cast<int>(t->rank);
    for (uint32_t d = 0; d < t->rank; ++d) { l.shape[d] = t->shape[d]; l.strides[d] = t->strides[d]; }
    return l;
}

}   // namespace

#define AIXB200_CTX() uint64_t launched_ = 0; kernels::LaunchContext ctx = makeContext(*this, &launched_)
#define AIXB200_DONE(what) do { m_stats.static_kernel_launches += launched_; m_stats.total_kernel_launches += launched_; checkLaunch(what); } while (0)

void Device::sum(const aixb200_tensor* a, const aixb200_tensor* r)
{
    View src = inputView(a, "sum");
    View dst = outputView(r, "sum");
    if (src.dtype != dst.dtype) failInvalid("sum: result must have the element type of the input");
    if (dst.size != 1) failInvalid("sum: result must have one element");
    if (recordReduction(Op::SumAll, src, dst)) return;
    flush();
    if (dryRun()) return;
    AIXB200_CTX();
    kernels::reduceAll(ctx, false, src, dst.firstByte());
    AIXB200_DONE("sum");
}

// A full reduction whose operand is the result of a recorded, not yet launched op is recorded too: the planner folds
// it into the producer's kernel, where the operand is still in registers.
bool Device::recordReduction(Op op, const View& src, const View& dst)
{
    if (!m_limits.fusion || !m_fuseReductions || src.size < 2) return false;
    bool producerPending = false;
    for (size_t i = m_pending.size(); i-- > 0 && !producerPending;)
        producerPending = m_pending[i].out.base == src.base && !isReduction(m_pending[i].op) && m_pending[i].out.sameElements(src);
    if (!producerPending) return false;
    OpRecord rec;
    rec.op = op;
    rec.numInputs = 1;
    rec.in[0] = src;
    rec.out = dst;
    record(std::move(rec));
    return true;
}

// reduceTo / maxTo over the trailing dimension of a dense [rows, cols] operand whose producer is still pending: recorded,
// so that the producing kernel folds every row while its elements are in registers (one warp or CTA per row) and the
// operand is not read back from memory. Rows must be plentiful enough to fill the GPU that way; anything else takes the
// stand-alone kernels.
bool Device::recordRowReduction(bool isMax, const View& src, const View& dst, uint64_t rows, uint64_t cols)
{
    if (!m_limits.fusion || !m_fuseReductions || !m_fuseRowReductions) return false;
    if (rows < static_cast<uint64_t>(m_smCount) * 4 || cols < 128 || !src.isDense() || !dst.isDense() || dst.size != rows) return false;
    bool producerPending = false;
    for (size_t i = m_pending.size(); i-- > 0 && !producerPending;)
        producerPending = !isReduction(m_pending[i].op) && m_pending[i].out.sameElements(src);
    if (!producerPending) return false;
    OpRecord rec;
    rec.op = isMax ? Op::MaxRows : Op::SumRows;
    rec.numInputs = 2;
    rec.in[0] = src;
    rec.in[1] = dst;
    rec.out = dst;
    rec.rowCols = cols;
    record(std::move(rec));
    return true;
}

// Sum for callers that must not allocate: no staging of host inputs, no flush of recorded work (a flush may
// compile and load a kernel), scratch in the library's static device array.
void Device::sumStaticScratch(const aixb200_tensor* a, const aixb200_tensor* r)
{
    if (dryRun()) failInvalid("sum_static_scratch needs a GPU");
    if (!m_pending.empty() || !m_deferredFrees.empty() || m_deferred.active)
        failInvalid("sum_static_scratch: recorded work is pending; call aixb200_synchronize() first (flushing here could allocate)");
    View src = makeView(a, "sum_static_scratch");
    View dst = makeView(r, "sum_static_scratch");
    if (src.dtype != dst.dtype) failInvalid("sum_static_scratch: result must have the element type of the input");
    if (dst.size != 1) failInvalid("sum_static_scratch: result must have one element");
    if (src.size > kernels::kStaticScratchMaxElements)
        failInvalid("sum_static_scratch: input has " + std::to_string(src.size) + " elements, the static scratch variant takes at most " +
                    std::to_string(kernels::kStaticScratchMaxElements));
    if (src.size == 0) failInvalid("sum_static_scratch: empty input");
    invalidatePreparedTerms(dst.firstByte(), dst.endByte());
    if ((!m_allocator->findBlock(src.base) && isHostPointer(src.base)) || (!m_allocator->findBlock(dst.base) && isHostPointer(dst.base)))
        failInvalid("sum_static_scratch: input and result must be device memory (host inputs would need a staging allocation)");
    // An overlapped all-reduce may still be working on the operand or the result: the device's stream waits for it, as
    // every other entry point does. Waiting on an event allocates nothing; the collective stays listed and is joined
    // again by the next ordinary call, which is harmless.
    for (const View* v : {&src, &dst})
    {
        const char* first = v->firstByte();
        const char* last = v->endByte();
        for (const CommInFlight& c : m_commInFlight)
            if (first < c.end && c.begin < last) check(cudaStreamWaitEvent(m_stream, c.done, 0), "cudaStreamWaitEvent(comm done)");
    }
    AIXB200_CTX();
    const char* error = kernels::sumWithStaticScratch(ctx, m_cfg.ordinal, src, dst.firstByte());
    m_stats.static_kernel_launches += launched_;
    m_stats.total_kernel_launches += launched_;
    if (error) failRuntime(std::string("sum_static_scratch: ") + error);
}

void Device::max(const aixb200_tensor* a, const aixb200_tensor* r)
{
    View src = inputView(a, "max");
    View dst = outputView(r, "max");
    if (src.dtype != dst.dtype) failInvalid("max: result must have the element type of the input");
    if (dst.size != 1 || src.size == 0) failInvalid("max: result must have one element and the input at least one");
    if (recordReduction(Op::MaxAll, src, dst)) return;
    flush();
    if (dryRun()) return;
    AIXB200_CTX();
    kernels::reduceAll(ctx, true, src, dst.firstByte());
    AIXB200_DONE("max");
}

void Device::argmax(const aixb200_tensor* a, const aixb200_tensor* r)
{
    View src = inputView(a, "argmax");
    View dst = outputView(r, "argmax");
    if (dst.dtype != I32) failInvalid("argmax supports only int32 data type for its result");
    flush();
    if (dryRun() || src.size == 0) return;
    AIXB200_CTX();
    kernels::argmaxAll(ctx, src, reinterpret_cast<int32_t*>(dst.firstByte()), false, src.size);
    AIXB200_DONE("argmax");
}

void Device::argmaxIndices(const aixb200_tensor* a, const aixb200_tensor* r)
{
    View src = inputView(a, "argmaxIndices");
    View dst = outputView(r, "argmaxIndices");
    if (dst.dtype != I32) failInvalid("argmaxIndices supports only int32 data type for its result");
    if (dst.size != src.size) failInvalid("argmaxIndices: result must have the size of the input");
    flush();
    if (dryRun() || src.size == 0) return;
    AIXB200_CTX();
    kernels::argmaxAll(ctx, src, reinterpret_cast<int32_t*>(dst.firstByte()), true, src.size);
    AIXB200_DONE("argmaxIndices");
}

// Pairs every source dimension with "kept" or "reduced" the way translationIndex does (aixDeviceCPU.cpp:627-649):
// walking both shapes from the back, a source dimension is kept when the destination has the same extent there.
static int classifyReduction(const aixb200_tensor* src, const aixb200_tensor* dst, kernels::ReduceDim* dims)
{
    int j = static_cast<int>(dst->rank) - 1;
    for (int i = static_cast<int>(src->rank) - 1; i >= 0; --i)
    {
        bool kept = false;
        if (j >= 0 && dst->shape[j] == src->shape[i]) { kept = true; --j; }
        else if (j >= 0 && dst->shape[j] == 1) { --j; }
        dims[i] = {src->shape[i], src->strides[i], kept};
    }
    // collapse: drop extent-1 dimensions, merge neighbours of the same kind whose strides chain
    int rank = 0;
    for (uint32_t i = 0; i < src->rank; ++i)
    {
        if (dims[i].extent == 1) continue;
        if (rank > 0 && dims[rank - 1].kept == dims[i].kept && dims[rank - 1].stride == dims[i].stride * dims[i].extent)
        {
            dims[rank - 1].extent *= dims[i].extent;
            dims[rank - 1].stride = dims[i].stride;
        }
        else dims[rank++] = dims[i];
    }
    return rank;
}

void Device::reduceTo(const aixb200_tensor* s, const aixb200_tensor* d, bool isMax)
{
    const char* what = isMax ? "maxTo" : "reduceTo";
    View src = inputView(s, what);
    View dst = outputView(d, what);
    if (src.dtype != dst.dtype) failInvalid(std::string(what) + ": element types differ");
    if (src.size == 0) { flush(); return; }
    kernels::ReduceDim dims[MAX_RANK];
    // inputView may have re-based a staged host tensor: the strides are unchanged, only base/offset moved.
    int rank = classifyReduction(s, d, dims);
    uint64_t outputs = 1;
    for (int i = 0; i < rank; ++i) if (dims[i].kept) outputs *= dims[i].extent;
    if (outputs != dst.size) failInvalid(std::string(what) + ": destination shape is not a reduction of the source shape");
    if (rank == 2 && dims[0].kept && !dims[1].kept && dims[1].stride == 1 && dims[0].stride == dims[1].extent &&
        recordRowReduction(isMax, src, dst, dims[0].extent, dims[1].extent))
        return;
    flush();
    if (dryRun()) return;
    // canonical 2-D forms need an explicit partner dimension
    kernels::ReduceDim two[2];
    const kernels::ReduceDim* use = dims;
    if (rank == 1)
    {
        if (dims[0].kept) { two[0] = dims[0]; two[1] = {1, 1, false}; }
        else              { two[0] = {1, 0, true}; two[1] = dims[0]; }
        use = two;
        rank = 2;
    }
    else if (rank == 0)
    {
        two[0] = {1, 0, true};
        two[1] = {1, 1, false};
        use = two;
        rank = 2;
    }
    AIXB200_CTX();
    kernels::reduceInto(ctx, isMax, src.dtype, src.firstByte(), use, rank, dst.firstByte());
    AIXB200_DONE(what);
}

void Device::argmaxTo(const aixb200_tensor* s, const aixb200_tensor* d, size_t dim, bool oneHot)
{
    const char* what = oneHot ? "argmaxIndicesTo" : "argmaxTo";
    View src = inputView(s, what);
    View dst = outputView(d, what);
    if (dst.dtype != I32) failInvalid(std::string(what) + " supports only int32 data type for its result");
    if (dim >= s->rank) failInvalid(std::string(what) + ": dimension out of range");
    flush();
    if (dryRun() || src.size == 0) return;
    kernels::ReduceDim dims[MAX_RANK];
    for (uint32_t i = 0; i < s->rank; ++i) dims[i] = {s->shape[i], s->strides[i], i != dim};
    AIXB200_CTX();
    kernels::argmaxAlong(ctx, src.dtype, src.firstByte(), dims, static_cast<int>(s->rank), static_cast<int>(dim),
                         reinterpret_cast<int32_t*>(dst.firstByte()), oneHot, src.size);
    AIXB200_DONE(what);
}

void Device::matmul(const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r)
{
    if (a->rank != 2 || b->rank != 2 || r->rank != 2) failInvalid("matmul: operands and result must be 2-D");
    if (a->shape[1] != b->shape[0] || r->shape[0] != a->shape[0] || r->shape[1] != b->shape[1]) failInvalid("matmul: shapes do not chain");
    if (a->dtype != r->dtype || b->dtype != r->dtype) failInvalid("matmul: element types differ");
    DeferredMatmul d;
    d.a = *a; d.b = *b; d.r = *r;
    d.va = inputView(a, "matmul"); d.vb = inputView(b, "matmul");
    d.vr = outputView(r, "matmul");
    flush();
    if (d.vr.size == 0) return;
    // Products whose consumers the kernel can fold wait for the ops that follow (see DeferredMatmul). Operands staged from
    // host memory live only until the next call, so those products are launched at once. A dry-run device goes through
    // the same decisions (and counts what it would have folded) without launching anything.
    if (m_foldMatmulEpilogue && m_staged.empty() && d.vr.isDense())
    {
        gemm::Problem probe{};
        probe.dtype = r->dtype;
        probe.m = a->shape[0]; probe.k = a->shape[1]; probe.n = b->shape[1];
        probe.c = d.vr.firstByte();
        probe.splitF32 = m_cfg.tf32x3_matmul != 0;
        if (gemm::canFoldEpilogue(probe, !dryRun())) { m_deferred = d; m_deferred.active = true; return; }
    }
    if (dryRun()) return;
    launchMatmul(d, 0);
}

void Device::launchMatmul(const DeferredMatmul& d, int folded, void* redirectTo)
{
    if (redirectTo)
    {
        // the zero-fill and the accumulation disappear: the product lands where their result would have
        m_pending.erase(m_pending.begin() + static_cast<std::ptrdiff_t>(std::max(d.addIndex, d.fillIndex)));
        m_pending.erase(m_pending.begin() + static_cast<std::ptrdiff_t>(std::min(d.addIndex, d.fillIndex)));
        m_stats.matmul_consumers_folded += 1;
        ++m_stats.fills_absorbed;
    }
    if (dryRun())
    {
        if (folded == 2) m_pending.erase(m_pending.begin() + static_cast<std::ptrdiff_t>(d.tanhIndex));
        if (folded >= 1) m_pending.erase(m_pending.begin() + static_cast<std::ptrdiff_t>(d.addIndex));
        m_stats.matmul_consumers_folded += static_cast<uint64_t>(folded);
        return;
    }
    const uint64_t m = d.a.shape[0], k = d.a.shape[1], n = d.b.shape[1];
    AIXB200_CTX();
    gemm::Problem p{};
    p.dtype = d.r.dtype;
    p.m = m; p.n = n; p.k = k;
    p.a = d.va.firstByte(); p.aRowStride = d.a.strides[0]; p.aColStride = d.a.strides[1];
    p.b = d.vb.firstByte(); p.bRowStride = d.b.strides[0]; p.bColStride = d.b.strides[1];
    p.c = redirectTo ? redirectTo : d.vr.firstByte();
    p.splitF32 = m_cfg.tf32x3_matmul != 0;
    p.shareDevice = !m_commInFlight.empty();
    int region = -1;
    if (folded > 0)
    {
        // exactly one output leaves the kernel: the sum, or its tanh (launchDeferredMatmul folds no further than that)
        p.bias = reinterpret_cast<const float*>(d.bias.firstByte());
        p.storeC = false;
        p.biasOut = folded == 2 ? nullptr : d.biasOut.firstByte();
        p.tanhOut = folded == 2 ? d.tanhOut.firstByte() : nullptr;
        // max|x| of that output for the matmul it will feed, as generated kernels leave it (appendOperandMaxEpilogues)
        const View& last = folded == 2 ? d.tanhOut : d.biasOut;
        const size_t bytes = static_cast<size_t>(last.endByte() - last.firstByte());
        if (m_termSlots && std::find(m_operandSizes.begin(), m_operandSizes.end(), bytes) != m_operandSizes.end())
            region = rememberOperandRegion(last.firstByte(), last.endByte(), false);
        if (region >= 0) p.maxSlot = preparedSlot(m_operandRegions[static_cast<size_t>(region)].slot);
    }
    const bool tensorCore = gemm::launchTensorCore(*this, ctx, p);
    if (tensorCore) m_checkErrorWord = true;
    else if (folded == 0)
        kernels::matmulSimt(ctx, d.r.dtype, p.a, p.aRowStride, p.aColStride, p.b, p.bRowStride, p.bColStride, p.c, m, n, k);
    (void)redirectTo;
    AIXB200_DONE("matmul");
    if (folded > 0 && !tensorCore) { launchMatmul(d, 0); return; }       // the consumers stay recorded and run as kernels
    if (folded > 0)
    {
        if (region >= 0) m_operandRegions[static_cast<size_t>(region)].fresh = true;
        if (folded == 2) m_pending.erase(m_pending.begin() + static_cast<std::ptrdiff_t>(d.tanhIndex));
        m_pending.erase(m_pending.begin() + static_cast<std::ptrdiff_t>(d.addIndex));
        m_stats.matmul_consumers_folded += static_cast<uint64_t>(folded);
    }
}

void Device::launchDeferredMatmul(bool consumerRecorded)
{
    const DeferredMatmul d = m_deferred;
    m_deferred = DeferredMatmul{};
    // A consumer is folded only when that leaves the kernel with ONE output: the value it consumes must be dead - its storage
    // deallocated and no other recorded op touching it. Measured on B200 (4096 x 4096 outputs): the product alone 83 us (K =
    // 1024); product, then add + tanh as a generated kernel 117 us; all three results written by the product's epilogue 135 us -
    // every CTA finishes its tile at the same moment, and a burst of three tiles per CTA cannot drain while the tensor
    // cores run the two chunks of K ahead that TMEM has room for. The tanh is not folded by default either (m_foldDepth):
    // with product and sum dead the separate kernel only reads one matrix and writes one (106.6 us for both launches),
    // while eight epilogue warps need about 5000 instructions per thread and tile for bias, tanh and the maximum (117.3 us).
    auto dead = [&](const View& v, size_t skipA, size_t skipB)
    {
        if (!m_released.count(v.base)) return false;
        for (size_t i = 0; i < m_pending.size(); ++i)
        {
            if (i == skipA || i == skipB) continue;
            const OpRecord& op = m_pending[i];
            if (op.out.overlaps(v)) return false;
            for (int q = 0; q < op.numInputs; ++q) if (op.in[q].overlaps(v)) return false;
        }
        return true;
    };
    // And the add alone is folded only when nothing recorded consumes the sum: a recorded consumer would run in one generated
    // kernel together with the add anyway, so folding saves no pass over memory there, while the folding instantiation is a
    // few microseconds slower than the plain one (98 against 83 us at K = 1024; 105 us for product + add kernel).
    if (d.redirect)
    {
        // `target = 0 + product` with the product dead: the product is written into the target itself (0 + x is x)
        const bool productDead = dead(d.vr, d.addIndex, d.addIndex);
        launchMatmul(d, 0, productDead ? d.biasOut.firstByte() : nullptr);
        for (const OpRecord& op : m_pending)
            if (op.out.overlaps(d.va) || op.out.overlaps(d.vb)) invalidatePreparedTerms(op.out.firstByte(), op.out.endByte());
        return;
    }
    int folded = d.folded;
    if (m_foldDepth < 2 && (folded == 2 || consumerRecorded)) folded = 0;
    if (folded == 2 && !dead(d.biasOut, d.addIndex, d.tanhIndex)) folded = 1;
    if (folded >= 1 && !dead(d.vr, d.addIndex, d.addIndex)) folded = 0;
    launchMatmul(d, folded);
    // Ops recorded while the product waited announced their writes (outputView) before the launch prepared the operands and
    // left the output's maximum: what they are going to overwrite is stale from their point in program order on.
    for (const OpRecord& op : m_pending)
        if (op.out.overlaps(d.va) || op.out.overlaps(d.vb) || (folded >= 1 && op.out.overlaps(d.biasOut)) || (folded == 2 && op.out.overlaps(d.tanhOut)))
            invalidatePreparedTerms(op.out.firstByte(), op.out.endByte());
}

void Device::advanceDeferredMatmul(size_t index)
{
    DeferredMatmul& d = m_deferred;
    const OpRecord& op = m_pending[index];
    auto touches = [](const OpRecord& o, const View& v)
    {
        if (o.out.overlaps(v)) return true;
        for (int q = 0; q < o.numInputs; ++q) if (o.in[q].overlaps(v)) return true;
        return false;
    };
    // The product is launched ahead of everything recorded: an output it writes must not be touched by an earlier recorded
    // op (one that stayed recorded across flushes), and its bias must not be written by one.
    auto untouchedBefore = [&](const View& v, size_t except)
    {
        for (size_t i = 0; i < index; ++i)
            if (i != except && touches(m_pending[i], v)) return false;
        return true;
    };
    auto denseLikeResult = [&](const View& v)
    {
        return v.dtype == F32 && v.isDense() && v.size == d.vr.size && reinterpret_cast<uintptr_t>(v.firstByte()) % 16 == 0 &&
               !v.overlaps(d.vr) && !v.overlaps(d.va) && !v.overlaps(d.vb);
    };
    if (d.redirect)
    {
        if (touches(op, d.biasOut) || touches(op, d.vr)) launchDeferredMatmul(true);
        return;
    }
    if (d.folded == 0)
    {
        if (!touches(op, d.vr)) return;                         // unrelated (a fill of some gradient, say): keep waiting
        const uint64_t m = d.r.shape[0], n = d.r.shape[1];
        auto isRowVector = [&](const View& v)
        {
            return v.dtype == F32 && v.rank == 2 && v.shape[0] == m && v.shape[1] == n && v.strides[0] == 0 && v.strides[1] == 1 &&
                   reinterpret_cast<uintptr_t>(v.firstByte()) % 16 == 0;
        };
        if (op.op == Op::Add && op.numInputs == 2 && denseLikeResult(op.out))
        {
            const int product = op.in[0].sameElements(d.vr) ? 0 : (op.in[1].sameElements(d.vr) ? 1 : -1);
            if (product >= 0 && isRowVector(op.in[1 - product]) && !op.in[1 - product].overlaps(op.out) && untouchedBefore(op.out, index))
            {
                bool biasWritten = false;
                for (size_t i = 0; i < index; ++i) biasWritten = biasWritten || m_pending[i].out.overlaps(op.in[1 - product]);
                if (!biasWritten)
                {
                    d.folded = 1;
                    d.addIndex = index;
                    d.bias = op.in[1 - product];
                    d.biasOut = op.out;
                    return;
                }
            }
        }
        // `target += result` where the target's zero-fill is still recorded and nothing else recorded touches the target:
        // a candidate for writing the product into the target directly (decided when the wait ends: the result must be dead)
        if (m_redirectMatmul && op.op == Op::Add && op.numInputs == 2 && denseLikeResult(op.out))
        {
            const int product = op.in[0].sameElements(d.vr) ? 0 : (op.in[1].sameElements(d.vr) ? 1 : -1);
            if (product >= 0 && op.in[1 - product].sameElements(op.out))
            {
                size_t fill = index;
                bool clean = true;
                for (size_t i = 0; i < index && clean; ++i)
                {
                    const OpRecord& other = m_pending[i];
                    if (!touches(other, op.out)) continue;
                    if (fill == index && other.op == Op::Fill && other.out.sameElements(op.out) && other.scalar.raw == 0) fill = i;
                    else clean = false;
                }
                if (clean && fill != index)
                {
                    d.redirect = true;
                    d.addIndex = index;
                    d.fillIndex = fill;
                    d.biasOut = op.out;
                    return;
                }
            }
        }
        launchDeferredMatmul();
        return;
    }
    if (d.folded == 2)
    {
        // both consumers are candidates; the call that recorded the tanh still held the sum, which is why the product was not
        // launched there and then: whether the sum is dead shows once that call has returned
        if (touches(op, d.tanhOut) || touches(op, d.biasOut)) launchDeferredMatmul(true);
        return;
    }
    if (!touches(op, d.biasOut)) return;
    if (op.op == Op::Tanh && op.numInputs == 1 && op.in[0].sameElements(d.biasOut) && denseLikeResult(op.out) && !op.out.overlaps(d.biasOut) &&
        !op.out.overlaps(d.bias) && untouchedBefore(op.out, d.addIndex))
    {
        d.folded = 2;
        d.tanhIndex = index;
        d.tanhOut = op.out;
        return;
    }
    launchDeferredMatmul(true);
}

void Device::transpose(const aixb200_tensor* a, const aixb200_tensor* r, size_t dim0, size_t dim1)
{
    View src = inputView(a, "transpose");
    View dst = outputView(r, "transpose");
    if (dim0 >= a->rank || dim1 >= a->rank) failInvalid("transpose: dimension out of range");
    if (src.dtype != dst.dtype || src.size != dst.size) failInvalid("transpose: result does not match the input");
    flush();
    if (dryRun() || src.size == 0) return;
    AIXB200_CTX();
    kernels::transposeGeneral(ctx, src.dtype, src.firstByte(), dst.firstByte(), src.size, layoutOf(a), layoutOf(r),
                              static_cast<int>(dim0), static_cast<int>(dim1));
    AIXB200_DONE("transpose");
}

void Device::copy(const void* src, uint32_t srcDtype, void* dst, uint32_t dstDtype, size_t count, bool immediate)
{
    const size_t ss = dtypeSize(srcDtype), ds = dtypeSize(dstDtype);
    if (count == 0) { if (immediate) synchronize(); return; }
    if (!src || !dst) failInvalid("copy: null pointer");
    noteCallRange(src, static_cast<const char*>(src) + count * ss);
    noteCallRange(dst, static_cast<char*>(dst) + count * ds);
    if (dryRun()) { flush(); return; }
    const bool srcHost = !m_allocator->findBlock(src) && isHostPointer(src);
    const bool dstHost = !m_allocator->findBlock(dst) && isHostPointer(dst);
    if (dstHost && !immediate) failInvalid("copy: result must have GPU memory (use copyImmediate to read back to the host)");

    aixb200_tensor ts{}, td{};
    ts.data = const_cast<void*>(src); ts.size = count; ts.dtype = srcDtype; ts.rank = 1; ts.shape[0] = count; ts.strides[0] = 1;
    td.data = dst; td.size = count; td.dtype = dstDtype; td.rank = 1; td.shape[0] = count; td.strides[0] = 1;
    if (!m_commInFlight.empty())
    {
        orderAfterCollectives(makeView(&ts, "copy"));      // plain memcpy paths below do not go through inputView / outputView
        orderAfterCollectives(makeView(&td, "copy"));
    }

    if (dstHost)
    {
        // device -> host read-back (extension over the reference, whose copy targets device memory only)
        if (srcHost) failInvalid("copy: source and destination are both host memory");
        const void* from = src;
        void* converted = nullptr;
        if (srcDtype != dstDtype)
        {
            converted = m_allocator->allocate(count * ds + 16);
            td.data = converted;
            OpRecord rec;
            rec.op = Op::Cast;
            rec.numInputs = 1;
            rec.in[0] = inputView(&ts, "copy");
            rec.out = makeView(&td, "copy");
            record(std::move(rec));
            from = converted;
        }
        flush();
        check(cudaMemcpyAsync(dst, from, count * ds, cudaMemcpyDeviceToHost, m_stream), "device-to-host copy");
        m_stats.d2h_bytes += count * ds;
        synchronize();
        if (converted) m_allocator->release(converted);
        return;
    }

    if (srcHost && srcDtype == dstDtype)
    {
        flush();                            // ops already recorded against dst must run first
        invalidatePreparedTerms(dst, static_cast<char*>(dst) + count * ds);
        check(cudaMemcpyAsync(dst, src, count * ss, cudaMemcpyHostToDevice, m_stream), "host-to-device copy");
        m_stats.h2d_bytes += count * ss;
    }
    else
    {
        // device source, or host source with conversion (staged by inputView): a Cast node that fuses like any op
        OpRecord rec;
        rec.op = Op::Cast;
        rec.numInputs = 1;
        rec.in[0] = inputView(&ts, "copy");
        rec.out = outputView(&td, "copy");
        record(std::move(rec));
    }
    if (immediate) synchronize();
}

void Device::contiguous(const aixb200_tensor* s, const aixb200_tensor* d)
{
    OpRecord rec;
    rec.op = Op::Cast;
    rec.numInputs = 1;
    rec.out = outputView(d, "contiguous");
    rec.in[0] = inputView(s, "contiguous");
    if (rec.in[0].dtype != rec.out.dtype) failInvalid("contiguous: element types differ");
    checkOperandSize(rec.in[0], rec.out, "contiguous");
    // A large transposed matrix made contiguous: as a recorded op it would become a generated kernel whose loads walk down
    // columns (one element per line); the tiled transpose kernel moves the same bytes through shared memory instead.
    const View& in = rec.in[0];
    if (!dryRun() && in.rank == 2 && in.strides[0] == 1 && in.strides[1] == in.shape[0] && in.shape[0] >= 64 && in.shape[1] >= 64 &&
        in.size >= (uint64_t(1) << 16) && rec.out.isDense() && !in.overlaps(rec.out))
    {
        flush();
        AIXB200_CTX();
        kernels::Layout source{}, result{};
        source.rank = result.rank = 2;
        source.shape[0] = in.shape[1]; source.shape[1] = in.shape[0]; source.strides[0] = in.shape[0]; source.strides[1] = 1;
        result.shape[0] = in.shape[0]; result.shape[1] = in.shape[1]; result.strides[0] = in.shape[1]; result.strides[1] = 1;
        kernels::transposeGeneral(ctx, in.dtype, in.firstByte(), rec.out.firstByte(), in.size, source, result, 0, 1);
        AIXB200_DONE("contiguous");
        return;
    }
    record(std::move(rec));
}

void Device::sliceSet(const aixb200_tensor* s, const aixb200_tensor* d, size_t dim, size_t start, size_t end, size_t step)
{
    View src = inputView(s, "sliceSet");
    View dst = outputView(d, "sliceSet");
    if (dim >= d->rank || step == 0 || end < start) failInvalid("sliceSet: bad slice");
    if (src.dtype != dst.dtype) failInvalid("sliceSet: element types differ");
    flush();
    if (dryRun() || src.size == 0) return;
    const uint64_t sliceExtent = (end - start + step - 1) / step;
    AIXB200_CTX();
    kernels::sliceSet(ctx, src.dtype, src.firstByte(), layoutOf(s), dst.firstByte(), layoutOf(d), src.size, static_cast<int>(dim), start, step, sliceExtent);
    AIXB200_DONE("sliceSet");
}

void Device::triangle(const aixb200_tensor* s, const aixb200_tensor* d, int64_t diagonal, bool lower)
{
    const char* what = lower ? "tril" : "triu";
    View src = inputView(s, what);
    View dst = outputView(d, what);
    if (s->rank < 2) failInvalid(std::string(what) + ": needs at least two dimensions");
    if (src.dtype != dst.dtype || src.size != dst.size) failInvalid(std::string(what) + ": result does not match the input");
    flush();
    if (dryRun() || src.size == 0) return;
    AIXB200_CTX();
    kernels::triangle(ctx, src.dtype, src.firstByte(), layoutOf(s), dst.firstByte(), layoutOf(d), dst.size, s->shape[s->rank - 2],
                      s->shape[s->rank - 1], diagonal, lower);
    AIXB200_DONE(what);
}

void Device::indexSelect(const aixb200_tensor* s, const aixb200_tensor* d, const aixb200_tensor* idx, size_t dim)
{
    View src = inputView(s, "indexSelect");
    View ind = inputView(idx, "indexSelect");
    View dst = outputView(d, "indexSelect");
    if (ind.dtype != I32) failInvalid("indexSelect: indices must be int32");
    if (src.dtype != dst.dtype) failInvalid("indexSelect: element types differ");
    if (s->rank != 0 && dim >= s->rank) failInvalid("indexSelect: dimension out of range");
    flush();
    if (dryRun() || dst.size == 0) return;
    uint64_t sliceSize = 1;
    for (size_t i = dim + 1; i < s->rank; ++i) sliceSize *= s->shape[i];
    const uint64_t dimSize = s->rank ? s->shape[dim] * sliceSize : 0;
    AIXB200_CTX();
    kernels::indexSelect(ctx, src.dtype, src.firstByte(), layoutOf(s), dst.firstByte(), reinterpret_cast<const int32_t*>(ind.firstByte()),
                         layoutOf(idx), ind.size, sliceSize, dimSize, dst.size);
    m_checkErrorWord = true;
    AIXB200_DONE("indexSelect");
}

void Device::indexAdd(const aixb200_tensor* s, const aixb200_tensor* d, const aixb200_tensor* idx, size_t dim)
{
    View src = inputView(s, "indexAdd");
    View ind = inputView(idx, "indexAdd");
    View dst = outputView(d, "indexAdd");
    if (ind.dtype != I32) failInvalid("indexAdd: indices must be int32");
    if (src.dtype != dst.dtype) failInvalid("indexAdd: element types differ");
    if (d->rank != 0 && dim >= d->rank) failInvalid("indexAdd: dimension out of range");
    flush();
    if (dryRun() || src.size == 0) return;
    uint64_t sliceSize = 1;
    for (size_t i = dim + 1; i < d->rank; ++i) sliceSize *= d->shape[i];
    const uint64_t dimSize = d->rank ? d->shape[dim] * sliceSize : 0;
    AIXB200_CTX();
    kernels::indexAdd(ctx, src.dtype, src.firstByte(), layoutOf(s), dst.firstByte(), reinterpret_cast<const int32_t*>(ind.firstByte()),
                      layoutOf(idx), ind.size, sliceSize, dimSize, src.size);
    m_checkErrorWord = true;
    AIXB200_DONE("indexAdd");
}

// ----------------------------------------------------------------------------------------------------------------
// timing helpers, statistics, communication
// ----------------------------------------------------------------------------------------------------------------
void Device::flushL2()
{
    flushAll();
    if (dryRun()) return;
    if (!m_l2Flush)
    {
        m_l2FlushBytes = size_t(256) << 20;       // twice the 126 MB L2
        check(cudaMalloc(&m_l2Flush, m_l2FlushBytes), "cudaMalloc(L2 flush buffer)");
    }
    AIXB200_CTX();
    kernels::flushL2(ctx, m_l2Flush, m_l2FlushBytes);
    AIXB200_DONE("flushL2");
}

void Device::selfTestBoundedWait(uint64_t limitNs)
{
    if (dryRun()) failInvalid("the bounded-wait self-test needs a GPU");
    flush();
    AIXB200_CTX();
    gemm::launchBoundedWaitSelfTest(ctx, limitNs);
    m_checkErrorWord = true;
    AIXB200_DONE("bounded-wait self-test");
}

void Device::fillStats(aixb200_stats* out) const
{
    *out = m_stats;
    out->bytes_in_use = m_allocator->bytesInUse();
    out->bytes_cached = m_allocator->bytesCached();
    out->bytes_reserved = m_allocator->bytesReserved();
    if (dryRun()) out->cuda_mallocs = m_allocator->rawAllocations();
}

void Device::commInit(int rank, int nranks, const void* id)
{
    if (dryRun() && !Comm::backendInjected()) failInvalid("communication needs a GPU");
    flush();
    m_comm.reset();
    m_comm = std::make_unique<Comm>(rank, nranks, id, m_cfg.ordinal);
}

// Whether a scale of 1/ranks is handed to the collective as its own averaging, or applied by a scaling pass after a
// plain sum. The blocking form averages inside the collective (a separate pass would sit on the critical path); the
// overlapped forms ask for a plain sum - the form NVSwitch can reduce in flight - and run the pass on the side stream,
// where it is hidden. AIXB200_COMM_AVG=1 / 0 forces one or the other.
static bool ncclAverages(bool overlapped)
{
    static const int forced = []{ const char* v = std::getenv("AIXB200_COMM_AVG"); return v ? (v[0] == '0' ? 0 : 1) : -1; }();
    return forced < 0 ? !overlapped : forced != 0;
}

void Device::allReduce(void* data, size_t count, uint32_t dtype, double scale)
{
    if (!m_comm) failInvalid("all_reduce: aixb200_comm_init was not called");
    noteCallRange(data, static_cast<char*>(data) + count * dtypeSize(dtype));
    flush();
    invalidatePreparedTerms(data, static_cast<char*>(data) + count * dtypeSize(dtype));
    commWait();                 // collectives of one communicator are issued in one order on every rank
    // A scale of exactly 1/ranks on a floating type is the collective's own averaging: no extra pass over the data.
    const bool average = ncclAverages(false) && isFloatType(dtype) && m_comm->size() > 1 && scale == 1.0 / m_comm->size();
    m_comm->allReduceSum(data, count, dtype, m_stream, average);
    if (scale != 1.0 && !average && !dryRun())
    {
        AIXB200_CTX();
        kernels::scaleInPlace(ctx, dtype, data, count, scale);
        AIXB200_DONE("all_reduce scale");
    }
}

// Overlapped form: the collective runs on a side stream, ordered after everything issued so far on the device's
// stream. Later work on the device's stream runs concurrently with it - except work that touches `data`: every op
// whose operands or result overlap a collective in flight is ordered after that collective (recorded work that does not
// depend on it is launched first). commWait() joins all collectives at once.
void Device::allReduceAsync(void* data, size_t count, uint32_t dtype, double scale)
{
    if (!m_comm) failInvalid("all_reduce_async: aixb200_comm_init was not called");
    const bool average = ncclAverages(true) && isFloatType(dtype) && m_comm->size() > 1 && scale == 1.0 / m_comm->size();
    startCollective(data, count, dtype, "all_reduce_async", [&](cudaStream_t)
    {
        m_comm->allReduceSum(data, count, dtype, m_commStream, average);
        if (scale != 1.0 && !average) scaleOnCommStream(data, count, dtype, scale);      // plain sum (the form in-switch reduction serves), then the pass
    });
}

// Reduce-scatter / all-gather pair of a sharded optimizer: after reduce_scatter_async rank r holds the (scaled) sum of
// slice r of `data` - the other slices hold unspecified partial data until an all_gather_async on the same buffer, which
// distributes every rank's slice to all. Both run on the side stream like all_reduce_async and are joined the same way.
void Device::reduceScatterAsync(void* data, size_t count, uint32_t dtype, double scale)
{
    if (!m_comm) failInvalid("reduce_scatter_async: aixb200_comm_init was not called");
    const size_t ranks = static_cast<size_t>(m_comm->size());
    if (count % ranks != 0) failInvalid("reduce_scatter_async: the element count must be a multiple of the number of ranks");
    const bool average = ncclAverages(true) && isFloatType(dtype) && ranks > 1 && scale == 1.0 / m_comm->size();
    startCollective(data, count, dtype, "reduce_scatter_async", [&](cudaStream_t)
    {
        if (ranks > 1) m_comm->reduceScatterSum(data, count, dtype, m_commStream, average);
        const size_t slice = count / ranks;
        if (scale != 1.0 && !average)
            scaleOnCommStream(static_cast<char*>(data) + static_cast<size_t>(m_comm->rank()) * slice * dtypeSize(dtype), slice, dtype, scale);
    });
}

void Device::allGatherAsync(void* data, size_t count, uint32_t dtype)
{
    if (!m_comm) failInvalid("all_gather_async: aixb200_comm_init was not called");
    const size_t ranks = static_cast<size_t>(m_comm->size());
    if (count % ranks != 0) failInvalid("all_gather_async: the element count must be a multiple of the number of ranks");
    // On the gather lane when the communicator has one: the parameters' all-gathers then overtake the reduce-scatters of the
    // last layers' gradients, which were issued earlier and are still running when the optimizer starts on the first layers.
    const bool ownLane = m_comm->hasGatherLane();
    startCollective(data, count, dtype, "all_gather_async", [&](cudaStream_t stream) { if (ranks > 1) m_comm->allGather(data, count, dtype, stream, ownLane); }, ownLane);
}

void Device::scaleOnCommStream(void* data, size_t count, uint32_t dtype, double scale)
{
    uint64_t launched = 0;
    kernels::LaunchContext ctx{m_commStream, m_smCount, m_scratch, m_scratchBytes, &launched};
    kernels::scaleInPlace(ctx, dtype, data, count, scale);
    m_stats.static_kernel_launches += launched; m_stats.total_kernel_launches += launched;
    checkLaunch("collective scale");
}

// Common frame of the overlapped collectives: order the side stream after everything issued so far on the device's
// stream, run `issue` there, and remember the buffer so that later ops touching it are ordered after the collective.
void Device::startCollective(void* data, size_t count, uint32_t dtype, const char* what, const std::function<void(cudaStream_t)>& issue, bool gatherLane)
{
    aixb200_tensor whole{};
    whole.data = data; whole.size = count; whole.dtype = dtype; whole.rank = 1; whole.shape[0] = count; whole.strides[0] = 1;
    const View range = makeView(&whole, what);
    noteCallRange(range.firstByte(), range.endByte());
    invalidatePreparedTerms(data, static_cast<char*>(data) + count * dtypeSize(dtype));
    if (!m_commInFlight.empty()) orderAfterCollectives(range);       // two collectives on one buffer keep their order
    flush();
    if (!m_commStream)
    {
        check(cudaStreamCreateWithFlags(&m_commStream, cudaStreamNonBlocking), "cudaStreamCreate(comm)");
        check(cudaEventCreateWithFlags(&m_commFork, cudaEventDisableTiming), "cudaEventCreate(comm)");
    }
    if (gatherLane && !m_gatherStream) check(cudaStreamCreateWithFlags(&m_gatherStream, cudaStreamNonBlocking), "cudaStreamCreate(gather)");
    const cudaStream_t side = gatherLane ? m_gatherStream : m_commStream;
    check(cudaEventRecord(m_commFork, m_stream), "cudaEventRecord(comm fork)");
    check(cudaStreamWaitEvent(side, m_commFork, 0), "cudaStreamWaitEvent(comm fork)");
    issue(side);
    cudaEvent_t done = nullptr;
    if (!m_commEventPool.empty()) { done = m_commEventPool.back(); m_commEventPool.pop_back(); }
    else check(cudaEventCreateWithFlags(&done, cudaEventDisableTiming), "cudaEventCreate(comm)");
    check(cudaEventRecord(done, side), "cudaEventRecord(comm done)");
    const char* begin = static_cast<const char*>(data);
    m_commInFlight.push_back({begin, begin + count * dtypeSize(dtype), done});
}

int Device::commRank() const { return m_comm ? m_comm->rank() : 0; }
int Device::commSize() const { return m_comm ? m_comm->size() : 1; }

void Device::orderAfterCollectives(const View& v)
{
    const char* first = static_cast<const char*>(v.firstByte());
    const char* last = first + v.span() * dtypeSize(v.dtype);
    bool flushed = false;
    for (size_t i = 0; i < m_commInFlight.size();)
    {
        const CommInFlight& c = m_commInFlight[i];
        if (first < c.end && c.begin < last)
        {
            // what is recorded so far does not depend on the collective: launch it first, then make the stream wait
            if (!flushed) { flush(); flushed = true; }
            check(cudaStreamWaitEvent(m_stream, c.done, 0), "cudaStreamWaitEvent(comm done)");
            m_commEventPool.push_back(c.done);
            m_commInFlight.erase(m_commInFlight.begin() + static_cast<std::ptrdiff_t>(i));
        }
        else ++i;
    }
}

// Joins only the collectives that touch [data, data + bytes): what an optimizer calls before it starts on one parameter,
// so that the join falls between two parameters' recorded ops instead of inside an expression.
void Device::commWaitFor(const void* data, size_t bytes)
{
    if (m_commInFlight.empty() || !data || bytes == 0) return;
    aixb200_tensor whole{};
    whole.data = const_cast<void*>(data); whole.size = bytes; whole.dtype = U8; whole.rank = 1; whole.shape[0] = bytes; whole.strides[0] = 1;
    noteCallRange(data, static_cast<const char*>(data) + bytes);
    orderAfterCollectives(makeView(&whole, "comm_wait_for"));
}

void Device::commWait()
{
    if (m_comm && !m_comm->aborted()) m_comm->checkAsyncError("comm_wait");      // a peer that died surfaces here instead of as a hang later
    for (const CommInFlight& c : m_commInFlight)
    {
        check(cudaStreamWaitEvent(m_stream, c.done, 0), "cudaStreamWaitEvent(comm done)");
        m_commEventPool.push_back(c.done);
    }
    m_commInFlight.clear();
}

void Device::commDestroy()
{
    if (m_comm)
    {
        commWait();
        cudaStreamSynchronize(m_stream);
        m_comm.reset();
    }
    if (m_gatherStream) { cudaStreamDestroy(m_gatherStream); m_gatherStream = nullptr; }
    if (m_commStream)
    {
        cudaStreamDestroy(m_commStream); cudaEventDestroy(m_commFork);
        for (cudaEvent_t e : m_commEventPool) cudaEventDestroy(e);
        m_commEventPool.clear();
        m_commStream = nullptr; m_commFork = nullptr;
    }
}

}   // namespace aixb200
