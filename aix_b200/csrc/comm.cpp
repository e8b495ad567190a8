#include "comm.hpp"

#include <cuda_runtime.h>
#include <dlfcn.h>

namespace aixb200
{

namespace
{

// Minimal slice of the NCCL C API (stable since NCCL 2.0).
typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
enum { kNcclSum = 0, kNcclAvg = 4 };
enum { kNcclInt32 = 2, kNcclInt64 = 4, kNcclHalf = 6, kNcclFloat = 7, kNcclDouble = 8, kNcclBfloat16 = 9 };

struct NcclApi
{
    int (*getUniqueId)(NcclUniqueId*) = nullptr;
    int (*commInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*commDestroy)(NcclComm) = nullptr;
    int (*allReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*reduceScatter)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*allGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*getErrorString)(int) = nullptr;
    void* handle = nullptr;
};

NcclApi& nccl()
{
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
    api.allReduce = reinterpret_cast<decltype(api.allReduce)>(sym("ncclAllReduce"));
    api.reduceScatter = reinterpret_cast<decltype(api.reduceScatter)>(sym("ncclReduceScatter"));
    api.allGather = reinterpret_cast<decltype(api.allGather)>(sym("ncclAllGather"));
    api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(sym("ncclGetErrorString"));
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

Comm::Comm(int rank, int nranks, const void* id128, int ordinal) : m_rank(rank), m_nranks(nranks)
{
    if (nranks < 1 || rank < 0 || rank >= nranks) failInvalid("comm_init: bad rank / nranks");
    NcclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    cudaSetDevice(ordinal);
    NcclComm comm = nullptr;
    checkNccl(nccl().commInitRank(&comm, nranks, id, rank), "ncclCommInitRank");
    m_comm = comm;
}

Comm::~Comm()
{
    if (m_comm) nccl().commDestroy(m_comm);
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
    checkNccl(nccl().allReduce(data, data, count, ncclType(dtype), average ? kNcclAvg : kNcclSum, m_comm, stream), "ncclAllReduce");
}

// In place: `data` holds count elements on every rank, count a multiple of the number of ranks; afterwards slice
// [rank * count / ranks, (rank + 1) * count / ranks) of this rank's buffer holds the sum (NCCL's in-place form: the
// receive buffer is the rank's own slice of the send buffer).
void Comm::reduceScatterSum(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool average)
{
    const size_t slice = count / static_cast<size_t>(m_nranks);
    char* own = static_cast<char*>(data) + static_cast<size_t>(m_rank) * slice * dtypeSize(dtype);
    checkNccl(nccl().reduceScatter(data, own, slice, ncclType(dtype), average ? kNcclAvg : kNcclSum, m_comm, stream), "ncclReduceScatter");
}

// In place: every rank contributes its own slice of `data` and receives all the others'.
void Comm::allGather(void* data, size_t count, uint32_t dtype, cudaStream_t stream)
{
    const size_t slice = count / static_cast<size_t>(m_nranks);
    const char* own = static_cast<const char*>(data) + static_cast<size_t>(m_rank) * slice * dtypeSize(dtype);
    checkNccl(nccl().allGather(own, data, slice, ncclType(dtype), m_comm, stream), "ncclAllGather");
}

}   // namespace aixb200
