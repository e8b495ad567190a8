#include "comm.hpp"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <thread>

#if __has_include(<nccl.h>)
#include <nccl.h>              // only for ncclConfig_t and its initializer (non-blocking initialisation)
#define AIXB200_HAVE_NCCL_CONFIG 1
#endif

namespace aixb200
{

namespace
{

// Minimal slice of the NCCL C API (stable since NCCL 2.0).
typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
enum { kNcclSum = 0, kNcclAvg = 4 };
enum { kNcclSuccess = 0, kNcclRemoteError = 6, kNcclInProgress = 7 };
enum { kNcclInt32 = 2, kNcclInt64 = 4, kNcclHalf = 6, kNcclFloat = 7, kNcclDouble = 8, kNcclBfloat16 = 9 };

constexpr int kDefaultMaxCtas = 0;       // see Comm::Comm

struct NcclApi
{
    int (*getUniqueId)(NcclUniqueId*) = nullptr;
    int (*commInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*commInitRankConfig)(NcclComm*, int, NcclUniqueId, int, void*) = nullptr;
    int (*commGetAsyncError)(NcclComm, int*) = nullptr;
    int (*commAbort)(NcclComm) = nullptr;
    int (*commDestroy)(NcclComm) = nullptr;
    int (*commSplit)(NcclComm, int, int, NcclComm*, void*) = nullptr;      // NCCL >= 2.18; optional
    int (*allReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*reduceScatter)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*allGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*getErrorString)(int) = nullptr;
    void* handle = nullptr;
};

// ---- injected back end for host-side tests of the failure paths: no library, no GPU, no network -------------------------
// mode 1: initialisation never completes (the communicator stays "in progress"); mode 2: initialisation and collectives
// succeed, and from the (errorAfterPolls + 1)-th status query on the communicator reports a remote error.
struct Injected { int mode = 0; int errorAfterPolls = 0; int inits = 0, polls = 0, aborts = 0, destroys = 0; };
Injected g_injected;
int fakeGetUniqueId(NcclUniqueId* id) { std::memset(id, 0, sizeof(*id)); return kNcclSuccess; }
int fakeInitRank(NcclComm* comm, int, NcclUniqueId, int) { ++g_injected.inits; *comm = &g_injected; return kNcclSuccess; }
int fakeInitRankConfig(NcclComm* comm, int, NcclUniqueId, int, void*)
{
    ++g_injected.inits;
    *comm = &g_injected;
    return g_injected.mode == 1 ? kNcclInProgress : kNcclSuccess;
}
int fakeGetAsyncError(NcclComm, int* state)
{
    ++g_injected.polls;
    *state = g_injected.mode == 1 ? kNcclInProgress : ((g_injected.mode == 2 && g_injected.polls > g_injected.errorAfterPolls) ? kNcclRemoteError : kNcclSuccess);
    return kNcclSuccess;
}
int fakeAbort(NcclComm) { ++g_injected.aborts; return kNcclSuccess; }
int fakeDestroy(NcclComm) { ++g_injected.destroys; return kNcclSuccess; }
int fakeAllReduce(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) { return kNcclSuccess; }
int fakeAllGather(const void*, void*, size_t, int, NcclComm, cudaStream_t) { return kNcclSuccess; }
const char* fakeErrorString(int code) { return code == kNcclRemoteError ? "remote process exited or there was a network error (injected)" : "injected back end"; }

NcclApi& nccl()
{
    static NcclApi fake;
    if (g_injected.mode != 0)
    {
        fake.getUniqueId = fakeGetUniqueId; fake.commInitRank = fakeInitRank; fake.commInitRankConfig = fakeInitRankConfig;
        fake.commGetAsyncError = fakeGetAsyncError; fake.commAbort = fakeAbort; fake.commDestroy = fakeDestroy;
        fake.allReduce = fakeAllReduce; fake.reduceScatter = fakeAllReduce; fake.allGather = fakeAllGather; fake.getErrorString = fakeErrorString;
        return fake;
    }
    static NcclApi api;
    if (api.handle) return api;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names)
    {
        api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) failRuntime("NCCL library (libnccl.so.2) could not be loaded");
    auto sym = [&](const char* name) { void* p = dlsym(api.handle, name); if (!p) failRuntime(std::string("NCCL symbol missing: ") + name); return p; };
    api.getUniqueId = reinterpret_cast<decltype(api.getUniqueId)>(sym("ncclGetUniqueId"));
    api.commInitRank = reinterpret_cast<decltype(api.commInitRank)>(sym("ncclCommInitRank"));
    api.commDestroy = reinterpret_cast<decltype(api.commDestroy)>(sym("ncclCommDestroy"));
    api.commInitRankConfig = reinterpret_cast<decltype(api.commInitRankConfig)>(sym("ncclCommInitRankConfig"));
    api.commGetAsyncError = reinterpret_cast<decltype(api.commGetAsyncError)>(sym("ncclCommGetAsyncError"));
    api.commAbort = reinterpret_cast<decltype(api.commAbort)>(sym("ncclCommAbort"));
    api.allReduce = reinterpret_cast<decltype(api.allReduce)>(sym("ncclAllReduce"));
    api.reduceScatter = reinterpret_cast<decltype(api.reduceScatter)>(sym("ncclReduceScatter"));
    api.allGather = reinterpret_cast<decltype(api.allGather)>(sym("ncclAllGather"));
    api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(sym("ncclGetErrorString"));
    api.commSplit = reinterpret_cast<decltype(api.commSplit)>(dlsym(api.handle, "ncclCommSplit"));
    return api;
}

void checkNccl(int r, const char* what)
{
    if (r != 0) failRuntime(std::string(what) + ": " + nccl().getErrorString(r));
}

}   // namespace

void Comm::uniqueId(void* out128)
{
    static_assert(sizeof(NcclUniqueId) == AIXB200_COMM_ID_BYTES, "id size");
    NcclUniqueId id;
    checkNccl(nccl().getUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out128, &id, sizeof(id));
}

void Comm::injectBackend(int mode, int errorAfterPolls)
{
    g_injected = Injected{};
    g_injected.mode = mode;
    g_injected.errorAfterPolls = errorAfterPolls;
}
bool Comm::backendInjected() { return g_injected.mode != 0; }
void Comm::injectedCounters(int* inits, int* polls, int* aborts)
{
    if (inits) *inits = g_injected.inits;
    if (polls) *polls = g_injected.polls;
    if (aborts) *aborts = g_injected.aborts;
}

// Blocking initialisation by default. With AIXB200_COMM_INIT_TIMEOUT_MS set, the communicator is created non-blocking
// (ncclCommInitRankConfig, config.blocking = 0) and polled with ncclCommGetAsyncError until it is ready or the deadline
// has passed - a rank that never joins then costs a timeout and an ncclCommAbort instead of a hang. A communicator created
// that way stays non-blocking: every later call may report "in progress" and is polled to completion the same way.
Comm::Comm(int rank, int nranks, const void* id128, int ordinal) : m_rank(rank), m_nranks(nranks)
{
    if (nranks < 1 || rank < 0 || rank >= nranks) failInvalid("comm_init: bad rank / nranks");
    NcclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    if (!backendInjected()) cudaSetDevice(ordinal);
    const char* limit = std::getenv("AIXB200_COMM_INIT_TIMEOUT_MS");
    m_timeoutMs = (limit && *limit) ? std::atol(limit) : 0;
    NcclComm comm = nullptr;
#ifdef AIXB200_HAVE_NCCL_CONFIG
    if (m_timeoutMs > 0)
    {
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.blocking = 0;
        m_nonBlocking = true;
        const int r = nccl().commInitRankConfig(&comm, nranks, id, rank, &config);
        m_comm = comm;
        if (r != kNcclSuccess && r != kNcclInProgress) { abortOnce(); checkNccl(r, "ncclCommInitRankConfig"); }
        waitUntilReady("ncclCommInitRankConfig");
        return;
    }
#endif
#ifdef AIXB200_HAVE_NCCL_CONFIG
    // AIXB200_COMM_MAX_CTAS: upper bound on the CTAs a collective's kernel may use. The collectives of the overlapped
    // exchange share the GPU with the matmuls of backward(); every SM they hold is one the persistent matmul grid cannot
    // start a CTA on. 0 leaves NCCL's own choice.
    const char* ctas = std::getenv("AIXB200_COMM_MAX_CTAS");
    const int maxCtas = (ctas && *ctas) ? std::atoi(ctas) : kDefaultMaxCtas;
    if (maxCtas > 0 && nccl().commInitRankConfig && !backendInjected())
    {
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.blocking = 1;
        config.maxCTAs = maxCtas;
        config.minCTAs = 1;
        checkNccl(nccl().commInitRankConfig(&comm, nranks, id, rank, &config), "ncclCommInitRankConfig");
    }
    else
#endif
    checkNccl(nccl().commInitRank(&comm, nranks, id, rank), "ncclCommInitRank");
    m_comm = comm;
    // A second communicator over the same ranks for the all-gathers of a sharded optimizer (see allGather;
    // AIXB200_COMM_GATHER_LANE=0: none). Every rank decides the same way: same library, same environment.
    const char* lane = std::getenv("AIXB200_COMM_GATHER_LANE");
    if (nranks > 1 && !backendInjected() && nccl().commSplit && !(lane && lane[0] == '0'))
    {
        NcclComm second = nullptr;
        checkNccl(nccl().commSplit(m_comm, 0, rank, &second, nullptr), "ncclCommSplit");
        m_gatherComm = second;
    }
}

Comm::~Comm()
{
    if (m_gatherComm && !m_aborted) nccl().commDestroy(m_gatherComm);
    if (m_comm && !m_aborted) nccl().commDestroy(m_comm);
}

void Comm::abortOnce()
{
    if (m_gatherComm && !m_aborted) nccl().commAbort(m_gatherComm);
    if (m_comm && !m_aborted) nccl().commAbort(m_comm);
    m_aborted = true;
}

// Polls the communicator's state until it leaves "in progress". A deadline that passes aborts the communicator and
// reports a timeout; an error state aborts it and reports the error.
void Comm::waitUntilReady(const char* what)
{
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(m_timeoutMs > 0 ? m_timeoutMs : 120000);
    for (;;)
    {
        int state = kNcclSuccess;
        const int r = nccl().commGetAsyncError(m_comm, &state);
        if (r != kNcclSuccess) { abortOnce(); checkNccl(r, "ncclCommGetAsyncError"); }
        if (state == kNcclSuccess) return;
        if (state != kNcclInProgress)
        {
            abortOnce();
            failRuntime(std::string(what) + ": asynchronous NCCL error: " + nccl().getErrorString(state) + "; the communicator was aborted");
        }
        if (std::chrono::steady_clock::now() > deadline)
        {
            abortOnce();
            throw Error(AIXB200_ERR_TIMEOUT, std::string(what) + " did not complete within " + std::to_string(m_timeoutMs > 0 ? m_timeoutMs : 120000) +
                                             " ms (a rank that never joined?); the communicator was aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

// One status query: an asynchronous error (a peer that died, a network fault) surfaces at the next call instead of as a
// hang in a later collective.
void Comm::checkAsyncError(const char* what)
{
    if (m_aborted) failRuntime(std::string(what) + ": the communicator was aborted after an earlier failure");
    int state = kNcclSuccess;
    if (nccl().commGetAsyncError(m_comm, &state) != kNcclSuccess) return;
    if (state == kNcclSuccess || state == kNcclInProgress) return;
    abortOnce();
    failRuntime(std::string(what) + ": asynchronous NCCL error: " + nccl().getErrorString(state) + "; the communicator was aborted");
}

void Comm::finishCall(int r, const char* what)
{
    if (r == kNcclInProgress && m_nonBlocking) { waitUntilReady(what); return; }
    checkNccl(r, what);
}

static int ncclType(uint32_t dtype)
{
    switch (dtype)
    {
        case F64: return kNcclDouble;
        case F32: return kNcclFloat;
        case F16: return kNcclHalf;
        case BF16: return kNcclBfloat16;
        case I64: return kNcclInt64;
        case I32: return kNcclInt32;
        default: failInvalid("collective: unsupported element type");
    }
}

void Comm::allReduceSum(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool average)
{
    checkAsyncError("all_reduce");
    finishCall(nccl().allReduce(data, data, count, ncclType(dtype), average ? kNcclAvg : kNcclSum, m_comm, stream), "ncclAllReduce");
}

// In place: `data` holds count elements on every rank, count a multiple of the number of ranks; afterwards slice
// [rank * count / ranks, (rank + 1) * count / ranks) of this rank's buffer holds the sum (NCCL's in-place form: the
// receive buffer is the rank's own slice of the send buffer).
void Comm::reduceScatterSum(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool average)
{
    const size_t slice = count / static_cast<size_t>(m_nranks);
    char* own = static_cast<char*>(data) + static_cast<size_t>(m_rank) * slice * dtypeSize(dtype);
    checkAsyncError("reduce_scatter");
    finishCall(nccl().reduceScatter(data, own, slice, ncclType(dtype), average ? kNcclAvg : kNcclSum, m_comm, stream), "ncclReduceScatter");
}

// In place: every rank contributes its own slice of `data` and receives all the others'.
void Comm::allGather(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool ownLane)
{
    const size_t slice = count / static_cast<size_t>(m_nranks);
    const char* own = static_cast<const char*>(data) + static_cast<size_t>(m_rank) * slice * dtypeSize(dtype);
    checkAsyncError("all_gather");
    finishCall(nccl().allGather(own, data, slice, ncclType(dtype), (ownLane && m_gatherComm) ? m_gatherComm : m_comm, stream), "ncclAllGather");
}

}   // namespace aixb200
