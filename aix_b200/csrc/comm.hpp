// Data-parallel exchange over NCCL (NVLink 5 / NVSwitch). The reference has no multi-device code; this exists for
// the data-parallel training configuration, where gradients are summed across the GPUs of one node.
// NCCL is opened with dlopen at first use so that the library loads on machines that have no NCCL or no GPU.
#pragma once

#include "common.hpp"

typedef struct CUstream_st* cudaStream_t;

namespace aixb200
{

class Comm
{
public:
    static void uniqueId(void* out128);
    Comm(int rank, int nranks, const void* id128, int ordinal);
    ~Comm();
    // Sum over the ranks; with `average` the sum is divided by the number of ranks inside the collective.
    void allReduceSum(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool average = false);
    void reduceScatterSum(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool average = false);
    // With `ownLane` the all-gather runs on a second communicator (split off the first one when the library offers
    // ncclCommSplit), so that on a stream of its own it does not queue behind reduce-scatters issued earlier: collectives of
    // one communicator run one after the other whatever streams they are given.
    void allGather(void* data, size_t count, uint32_t dtype, cudaStream_t stream, bool ownLane = false);
    bool hasGatherLane() const { return m_gatherComm != nullptr; }
    int rank() const { return m_rank; }
    int size() const { return m_nranks; }
    // One query of the communicator's asynchronous state; an error aborts the communicator (once) and throws.
    void checkAsyncError(const char* what);
    bool aborted() const { return m_aborted; }

    // Host-side fault injection (tests): replaces the NCCL entry points by stand-ins. mode 0 restores NCCL.
    static void injectBackend(int mode, int errorAfterPolls);
    static bool backendInjected();
    static void injectedCounters(int* inits, int* polls, int* aborts);

private:
    void waitUntilReady(const char* what);
    void finishCall(int result, const char* what);
    void abortOnce();
    void* m_comm = nullptr;
    void* m_gatherComm = nullptr;   // second communicator over the same ranks, for all-gathers (AIXB200_COMM_GATHER_LANE=0: none)
    int   m_rank, m_nranks;
    long  m_timeoutMs = 0;
    bool  m_nonBlocking = false, m_aborted = false;
};

}   // namespace aixb200
