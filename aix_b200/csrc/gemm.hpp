// Tensor-core GEMM entry (tcgen05 / TMEM / TMA, sm_100a).
#pragma once

#include "kernels.hpp"

namespace aixb200
{
class Device;
}

namespace aixb200::gemm
{

// C[m,n] (dense, row-major) = A[m,k] . B[k,n]; A and B are addressed as base[row * rowStride + col * colStride].
struct Problem
{
    uint32_t    dtype;
    uint64_t    m, n, k;
    const void* a; uint64_t aRowStride, aColStride;
    const void* b; uint64_t bRowStride, bColStride;
    void*       c;
    bool        splitF32;      // f32 operands: three-pass split so that the result keeps f32 accuracy
    bool        shareDevice;   // another stream of this device has kernels in flight (a collective): leave it some SMs
    // Elementwise consumers folded into the epilogue of the f32 kernel (nn::Linear is matmul(x, W) + b, usually followed by
    // tanh: aixNeuralNetwork.hpp:150-153). `bias` set: the kernel also writes C + bias (row vector of n values) to biasOut
    // and / or tanh(C + bias) to tanhOut, both dense m x n like C, from the registers that hold the finished tile; C itself
    // is written only if storeC. maxSlot receives the bit pattern of max|x| of the last of these outputs (the next
    // matmul's operand). launchTensorCore returns false, having launched no product, when it cannot do this.
    const float* bias = nullptr;
    void*       biasOut = nullptr;
    void*       tanhOut = nullptr;
    bool        storeC = true;
    uint32_t*   maxSlot = nullptr;
};

// Whether launchTensorCore would fold the problem's consumers (pointers, shape and element type decide; operands do not).
// needDriver = false leaves out the check that the driver's tensor-map encoder can be reached (dry-run devices).
bool canFoldEpilogue(const Problem& problem, bool needDriver = true);

// Runs the problem on the tensor cores when its element type, shape and alignment allow it.
// Returns false (having launched nothing) when the caller must use the CUDA-core kernel instead.
bool launchTensorCore(Device& device, const kernels::LaunchContext& ctx, const Problem& problem);

// One tiny kernel that waits, with the matmul's own bounded-wait routine, on an mbarrier nobody arrives at, gives up after
// limitNs and raises the device's error word (LaunchContext::scratch + kScratchTimeoutOffset). No TMA, no tensor-core work.
void launchBoundedWaitSelfTest(const kernels::LaunchContext& ctx, uint64_t limitNs);

}   // namespace aixb200::gemm
