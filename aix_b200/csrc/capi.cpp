// extern "C" surface of the B200 device (include/aixb200.h). Every function converts exceptions into status codes.
#include "comm.hpp"
#include "device.hpp"

#include <cuda_runtime.h>

#include <mutex>

using namespace aixb200;

struct aixb200_device
{
    std::unique_ptr<Device> impl;
    std::string error;
};

struct aixb200_event
{
    cudaEvent_t event = nullptr;
};

namespace
{

std::string g_createError;

template <class F>
int guarded(aixb200_device* dev, F&& body)
{
    if (!dev || !dev->impl) return AIXB200_ERR_INVALID;
    try
    {
        if (!dev->impl->dryRun()) cudaSetDevice(dev->impl->ordinal());
        dev->impl->beginCall();
        body(*dev->impl);
        return AIXB200_OK;
    }
    catch (const Error& e) { dev->error = e.what(); return e.code; }
    catch (const std::exception& e) { dev->error = e.what(); return AIXB200_ERR_RUNTIME; }
}

}   // namespace

extern "C"
{

void aixb200_default_config(aixb200_config* cfg)
{
    if (!cfg) return;
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->flush_threshold = 200;
    cfg->strict_math = 0;
    cfg->fusion = 1;
    cfg->disk_cache = 1;
    cfg->tf32x3_matmul = 1;
}

int aixb200_create(int ordinal, aixb200_device** out)
{
    aixb200_config cfg;
    aixb200_default_config(&cfg);
    cfg.ordinal = ordinal;
    return aixb200_create_with_config(&cfg, out);
}

int aixb200_create_with_config(const aixb200_config* cfg, aixb200_device** out)
{
    if (!cfg || !out) { g_createError = "null argument"; return AIXB200_ERR_INVALID; }
    *out = nullptr;
    try
    {
        auto dev = std::make_unique<aixb200_device>();
        dev->impl = std::make_unique<Device>(*cfg);
        *out = dev.release();
        return AIXB200_OK;
    }
    catch (const Error& e) { g_createError = e.what(); return e.code; }
    catch (const std::exception& e) { g_createError = e.what(); return AIXB200_ERR_RUNTIME; }
}

void aixb200_destroy(aixb200_device* dev)
{
    if (!dev) return;
    if (dev->impl && !dev->impl->dryRun()) cudaSetDevice(dev->impl->ordinal());
    delete dev;
}

const char* aixb200_last_error(const aixb200_device* dev) { return dev ? dev->error.c_str() : g_createError.c_str(); }
const char* aixb200_name(const aixb200_device* dev) { return (dev && dev->impl) ? dev->impl->name().c_str() : ""; }
const char* aixb200_version(void) { return "0.1.0"; }

int aixb200_device_count(void)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return 0; }
    return count;
}

int aixb200_allocate(aixb200_device* dev, size_t bytes, void** out)
{
    if (!out) return AIXB200_ERR_INVALID;
    return guarded(dev, [&](Device& d) { *out = d.allocate(bytes); });
}

int aixb200_allocate_typed(aixb200_device* dev, size_t count, uint32_t dtype, void** out)
{
    if (!out) return AIXB200_ERR_INVALID;
    return guarded(dev, [&](Device& d) { *out = d.allocate(count * dtypeSize(dtype)); });
}

int aixb200_deallocate(aixb200_device* dev, void* memory) { return guarded(dev, [&](Device& d) { d.deallocate(memory); }); }
int aixb200_empty_cache(aixb200_device* dev) { return guarded(dev, [&](Device& d) { d.emptyCache(); }); }
int aixb200_synchronize(aixb200_device* dev) { return guarded(dev, [&](Device& d) { d.synchronize(); }); }

#define AIXB200_BINARY(NAME, OP)                                                                                       \
    int aixb200_##NAME(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r)  \
    { return guarded(dev, [&](Device& d) { d.recordBinary(Op::OP, a, b, r, #NAME); }); }
#define AIXB200_UNARY(NAME, OP)                                                                                        \
    int aixb200_##NAME(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r)                           \
    { return guarded(dev, [&](Device& d) { d.recordUnary(Op::OP, a, r, #NAME); }); }

AIXB200_BINARY(add, Add)
AIXB200_BINARY(sub, Sub)
AIXB200_BINARY(mul, Mul)
AIXB200_BINARY(div, Div)
AIXB200_BINARY(pow, Pow)
AIXB200_UNARY(unary, Neg)
AIXB200_UNARY(sqrt, Sqrt)
AIXB200_UNARY(sin, Sin)
AIXB200_UNARY(cos, Cos)
AIXB200_UNARY(tanh, Tanh)
AIXB200_UNARY(log, Log)
AIXB200_UNARY(exp, Exp)

int aixb200_fill(aixb200_device* dev, const void* scalar, uint32_t scalarDtype, const aixb200_tensor* r)
{ return guarded(dev, [&](Device& d) { d.recordFill(scalar, scalarDtype, r); }); }
int aixb200_fill_min(aixb200_device* dev, const aixb200_tensor* r) { return guarded(dev, [&](Device& d) { d.recordFillMin(r); }); }

int aixb200_sum(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r) { return guarded(dev, [&](Device& d) { d.sum(a, r); }); }
int aixb200_sum_static_scratch(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r)
{ return guarded(dev, [&](Device& d) { d.sumStaticScratch(a, r); }); }
int aixb200_max(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r) { return guarded(dev, [&](Device& d) { d.max(a, r); }); }
int aixb200_argmax(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r) { return guarded(dev, [&](Device& d) { d.argmax(a, r); }); }
int aixb200_argmax_indices(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r)
{ return guarded(dev, [&](Device& d) { d.argmaxIndices(a, r); }); }
int aixb200_reduce_to(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t) { return guarded(dev, [&](Device& d) { d.reduceTo(s, t, false); }); }
int aixb200_max_to(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t) { return guarded(dev, [&](Device& d) { d.reduceTo(s, t, true); }); }
int aixb200_argmax_to(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, size_t dim)
{ return guarded(dev, [&](Device& d) { d.argmaxTo(s, t, dim, false); }); }
int aixb200_argmax_indices_to(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, size_t dim)
{ return guarded(dev, [&](Device& d) { d.argmaxTo(s, t, dim, true); }); }

int aixb200_matmul(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r)
{ return guarded(dev, [&](Device& d) { if (!a || !b || !r) failInvalid("matmul: null tensor descriptor"); d.matmul(a, b, r); }); }

int aixb200_transpose(aixb200_device* dev, const aixb200_tensor* a, const aixb200_tensor* r, size_t dim0, size_t dim1)
{ return guarded(dev, [&](Device& d) { d.transpose(a, r, dim0, dim1); }); }
int aixb200_copy(aixb200_device* dev, const void* src, uint32_t sdt, void* dst, uint32_t ddt, size_t count)
{ return guarded(dev, [&](Device& d) { d.copy(src, sdt, dst, ddt, count, false); }); }
int aixb200_copy_immediate(aixb200_device* dev, const void* src, uint32_t sdt, void* dst, uint32_t ddt, size_t count)
{ return guarded(dev, [&](Device& d) { d.copy(src, sdt, dst, ddt, count, true); }); }
int aixb200_contiguous(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t) { return guarded(dev, [&](Device& d) { d.contiguous(s, t); }); }
int aixb200_slice_set(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, size_t dim, size_t start, size_t end, size_t step)
{ return guarded(dev, [&](Device& d) { d.sliceSet(s, t, dim, start, end, step); }); }
int aixb200_tril(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, int64_t diagonal)
{ return guarded(dev, [&](Device& d) { d.triangle(s, t, diagonal, true); }); }
int aixb200_triu(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, int64_t diagonal)
{ return guarded(dev, [&](Device& d) { d.triangle(s, t, diagonal, false); }); }
int aixb200_index_select(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, const aixb200_tensor* idx, size_t dim)
{ return guarded(dev, [&](Device& d) { d.indexSelect(s, t, idx, dim); }); }
int aixb200_index_add(aixb200_device* dev, const aixb200_tensor* s, const aixb200_tensor* t, const aixb200_tensor* idx, size_t dim)
{ return guarded(dev, [&](Device& d) { d.indexAdd(s, t, idx, dim); }); }

int aixb200_get_stats(aixb200_device* dev, aixb200_stats* out)
{
    if (!out) return AIXB200_ERR_INVALID;
    return guarded(dev, [&](Device& d) { d.fillStats(out); });
}

const char* aixb200_last_kernel_source(const aixb200_device* dev) { return (dev && dev->impl) ? dev->impl->lastKernelSource() : nullptr; }

int aixb200_event_create(aixb200_device* dev, aixb200_event** out)
{
    if (!out) return AIXB200_ERR_INVALID;
    return guarded(dev, [&](Device& d)
    {
        if (d.dryRun()) failInvalid("events need a GPU");
        auto ev = new aixb200_event();
        if (cudaEventCreate(&ev->event) != cudaSuccess) { delete ev; failRuntime("cudaEventCreate failed"); }
        *out = ev;
    });
}

int aixb200_event_record(aixb200_device* dev, aixb200_event* ev)
{
    return guarded(dev, [&](Device& d)
    {
        if (!ev) failInvalid("null event");
        d.flushAll();
        if (cudaEventRecord(ev->event, d.stream()) != cudaSuccess) failRuntime("cudaEventRecord failed");
    });
}

int aixb200_event_elapsed_ms(aixb200_device* dev, aixb200_event* start, aixb200_event* stop, float* ms)
{
    return guarded(dev, [&](Device&)
    {
        if (!start || !stop || !ms) failInvalid("null argument");
        if (cudaEventSynchronize(stop->event) != cudaSuccess) failRuntime("cudaEventSynchronize failed");
        if (cudaEventElapsedTime(ms, start->event, stop->event) != cudaSuccess) failRuntime("cudaEventElapsedTime failed");
    });
}

int aixb200_event_destroy(aixb200_device* dev, aixb200_event* ev)
{
    return guarded(dev, [&](Device&) { if (ev) { cudaEventDestroy(ev->event); delete ev; } });
}

int aixb200_flush_l2(aixb200_device* dev) { return guarded(dev, [&](Device& d) { d.flushL2(); }); }
int aixb200_self_test_bounded_wait(aixb200_device* dev, uint64_t limitNs) { return guarded(dev, [&](Device& d) { d.selfTestBoundedWait(limitNs); }); }

int aixb200_comm_unique_id(void* idOut)
{
    if (!idOut) return AIXB200_ERR_INVALID;
    try { Comm::uniqueId(idOut); return AIXB200_OK; }
    catch (const Error& e) { g_createError = e.what(); return e.code; }
    catch (const std::exception& e) { g_createError = e.what(); return AIXB200_ERR_RUNTIME; }
}

int aixb200_comm_init(aixb200_device* dev, int rank, int nranks, const void* id)
{ return guarded(dev, [&](Device& d) { if (!id) failInvalid("null id"); d.commInit(rank, nranks, id); }); }
int aixb200_all_reduce(aixb200_device* dev, void* data, size_t count, uint32_t dtype, double scale)
{ return guarded(dev, [&](Device& d) { d.allReduce(data, count, dtype, scale); }); }
int aixb200_all_reduce_async(aixb200_device* dev, void* data, size_t count, uint32_t dtype, double scale)
{ return guarded(dev, [&](Device& d) { d.allReduceAsync(data, count, dtype, scale); }); }
int aixb200_reduce_scatter_async(aixb200_device* dev, void* data, size_t count, uint32_t dtype, double scale)
{ return guarded(dev, [&](Device& d) { d.reduceScatterAsync(data, count, dtype, scale); }); }
int aixb200_all_gather_async(aixb200_device* dev, void* data, size_t count, uint32_t dtype)
{ return guarded(dev, [&](Device& d) { d.allGatherAsync(data, count, dtype); }); }
int aixb200_comm_rank(aixb200_device* dev, int* rank, int* nranks)
{ return guarded(dev, [&](Device& d) { if (rank) *rank = d.commRank(); if (nranks) *nranks = d.commSize(); }); }
int aixb200_comm_inject_backend(int mode, int errorAfterPolls)
{
    if (mode < 0 || mode > 2) return AIXB200_ERR_INVALID;
    Comm::injectBackend(mode, errorAfterPolls);
    return AIXB200_OK;
}
int aixb200_comm_injected_counters(int* inits, int* polls, int* aborts) { Comm::injectedCounters(inits, polls, aborts); return AIXB200_OK; }
int aixb200_comm_wait(aixb200_device* dev) { return guarded(dev, [&](Device& d) { d.commWait(); }); }
int aixb200_comm_wait_for(aixb200_device* dev, const void* data, size_t bytes)
{ return guarded(dev, [&](Device& d) { d.commWaitFor(data, bytes); }); }
int aixb200_comm_destroy(aixb200_device* dev) { return guarded(dev, [&](Device& d) { d.commDestroy(); }); }

}   // extern "C"
