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

void Comm::allReduceSum(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool average)
{
    int type;
    switch (dtype)
    {
        case F64: type = kNcclDouble; break;
        case F32: type = kNcclFloat; break;
        case F16: type = kNcclHalf; break;
        case BF16: type = kNcclBfloat16; break;
        case I64: type = kNcclInt64; break;
        case I32: type = kNcclInt32; break;
        default: failInvalid("all_reduce: unsupported element type");
    }
    checkNccl(nccl().allReduce(data, data, count, type, average ? kNcclAvg : kNcclSum, m_comm, stream), "ncclAllReduce");
}

}   // namespace aixb200
