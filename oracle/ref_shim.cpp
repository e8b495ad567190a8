// TEST INFRASTRUCTURE - not part of the product.
//
// C ABI over the reference's own CPU device (aix::DeviceCPU, Targets/AIXLib/aixDeviceCPU.cpp), so that the
// parity tests and the CPU-baseline leg of the benchmark can drive the unmodified reference implementation with
// the same POD tensor descriptors the B200 library takes. This file contains no arithmetic of its own: every
// entry point converts descriptors and forwards to the reference method of the same name. It is compiled
// together with the reference's sources (taken where they lie, never copied) by oracle/build_ref.py into
// oracle/_ref/libaixref.so.
#include "aix.hpp"
#include "../include/aixb200.h"

#include <chrono>
#include <cstring>

namespace
{

aix::DeviceCPU& cpu()
{
    static aix::DeviceCPU device;
    return device;
}

aix::DeviceTensorParams toParams(const aixb200_tensor* t)
{
    aix::DeviceTensorParams p;
    p.data   = t->data;
    p.dtype  = static_cast<aix::DataType>(t->dtype);
    p.offset = t->offset;
    p.size   = t->size;
    p.shape.assign(t->shape, t->shape + t->rank);
    p.strides.assign(t->strides, t->strides + t->rank);
    // Same rule as TensorValue::computeIsContiguous (aixCore.hpp:1471-1480): strides equal the canonical ones.
    bool contiguous = true;
    size_t expected = 1;
    for (size_t i = t->rank; i-- > 0;)
    {
        if (p.strides[i] != expected) { contiguous = false; break; }
        expected *= p.shape[i];
    }
    p.isContiguous = contiguous;
    return p;
}

}   // namespace

#define AIXREF_BINARY(NAME, METHOD)                                                                                   \
    extern "C" int aixref_##NAME(const aixb200_tensor* a, const aixb200_tensor* b, const aixb200_tensor* r)          \
    { cpu().METHOD(toParams(a), toParams(b), toParams(r)); return 0; }
#define AIXREF_UNARY(NAME, METHOD)                                                                                    \
    extern "C" int aixref_##NAME(const aixb200_tensor* a, const aixb200_tensor* r)                                   \
    { cpu().METHOD(toParams(a), toParams(r)); return 0; }

AIXREF_BINARY(add, add)
AIXREF_BINARY(sub, sub)
AIXREF_BINARY(mul, mul)
AIXREF_BINARY(div, div)
AIXREF_BINARY(pow, pow)
AIXREF_BINARY(matmul, matmul)
AIXREF_UNARY(unary, unary)
AIXREF_UNARY(sqrt, sqrt)
AIXREF_UNARY(sin, sin)
AIXREF_UNARY(cos, cos)
AIXREF_UNARY(tanh, tanh)
AIXREF_UNARY(log, log)
AIXREF_UNARY(exp, exp)
AIXREF_UNARY(sum, sum)
AIXREF_UNARY(max, max)
AIXREF_UNARY(argmax, argmax)
AIXREF_UNARY(argmax_indices, argmaxIndices)
AIXREF_UNARY(contiguous, contiguous)
AIXREF_UNARY(reduce_to, reduceTo)
AIXREF_UNARY(max_to, maxTo)

extern "C"
{

void* aixref_allocate(size_t bytes)   { return cpu().allocate(bytes); }
void  aixref_deallocate(void* memory) { cpu().deallocate(memory); }

int aixref_fill(const void* scalar, uint32_t scalarDType, const aixb200_tensor* r)
{
    cpu().fill(scalar, static_cast<aix::DataType>(scalarDType), toParams(r));
    return 0;
}

int aixref_fill_min(const aixb200_tensor* r) { cpu().fillMin(toParams(r)); return 0; }

int aixref_copy(const void* src, uint32_t srcDType, void* dst, uint32_t dstDType, size_t count)
{
    cpu().copy(src, static_cast<aix::DataType>(srcDType), dst, static_cast<aix::DataType>(dstDType), count);
    return 0;
}

int aixref_transpose(const aixb200_tensor* a, const aixb200_tensor* r, size_t dim0, size_t dim1)
{
    cpu().transpose(toParams(a), toParams(r), dim0, dim1);
    return 0;
}

int aixref_argmax_to(const aixb200_tensor* s, const aixb200_tensor* d, size_t dim)
{
    cpu().argmaxTo(toParams(s), toParams(d), dim);
    return 0;
}

int aixref_argmax_indices_to(const aixb200_tensor* s, const aixb200_tensor* d, size_t dim)
{
    cpu().argmaxIndicesTo(toParams(s), toParams(d), dim);
    return 0;
}

int aixref_slice_set(const aixb200_tensor* s, const aixb200_tensor* d, size_t dim, size_t start, size_t end, size_t step)
{
    cpu().sliceSet(toParams(s), toParams(d), dim, start, end, step);
    return 0;
}

int aixref_tril(const aixb200_tensor* s, const aixb200_tensor* d, int64_t diagonal)
{
    cpu().tril(toParams(s), toParams(d), static_cast<ssize_t>(diagonal));
    return 0;
}

int aixref_triu(const aixb200_tensor* s, const aixb200_tensor* d, int64_t diagonal)
{
    cpu().triu(toParams(s), toParams(d), static_cast<ssize_t>(diagonal));
    return 0;
}

int aixref_index_select(const aixb200_tensor* s, const aixb200_tensor* d, const aixb200_tensor* idx, size_t dim)
{
    cpu().indexSelect(toParams(s), toParams(d), toParams(idx), dim);
    return 0;
}

int aixref_index_add(const aixb200_tensor* s, const aixb200_tensor* d, const aixb200_tensor* idx, size_t dim)
{
    cpu().indexAdd(toParams(s), toParams(d), toParams(idx), dim);
    return 0;
}

size_t aixref_dtype_size(uint32_t dtype) { return aix::Device::dataTypeSize(static_cast<aix::DataType>(dtype)); }

// ---------------------------------------------------------------------------------------------------------------
// Whole-path drivers through the reference's own front end (aix::Tensor / autograd / nn / optim on DeviceCPU).
// They exist so that golden vectors and the timed CPU baseline come from the reference's public API rather than
// from a hand-rolled op sequence.
// ---------------------------------------------------------------------------------------------------------------

// z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c)); returns z (n floats) and its sum; seconds = CPU time of the
// expression and the sum (inputs already built). a, b, c are n = rows*cols floats.
double aixref_chain_f32(const float* a, const float* b, const float* c, size_t rows, size_t cols, float* z, float* sum)
{
    using namespace aix;
    Shape shape{rows, cols};
    size_t n = rows * cols;
    auto ta = Tensor(a, n, DataType::kFloat32, shape);
    auto tb = Tensor(b, n, DataType::kFloat32, shape);
    auto tc = Tensor(c, n, DataType::kFloat32, shape);
    auto t0 = std::chrono::steady_clock::now();
    auto tz = (ta * tb + tc) * (1 / (1 + (-ta).exp())) - tb.tanh() / (1 + (-tc).exp());
    auto ts = tz.sum();
    auto t1 = std::chrono::steady_clock::now();
    if (z)   std::memcpy(z, tz.value().data(), n * sizeof(float));
    if (sum) *sum = ts.value().item<float>();
    return std::chrono::duration<double>(t1 - t0).count();
}

// One MLP data-parallel replica on the CPU device: layer widths dims[0..nLayers], tanh between layers, MSE loss,
// Adam(lr, 0.9, 0.999, 1e-8). Weights (in x out, row-major) and biases (1 x out) are given explicitly and updated
// in place; x is batch x dims[0], y is batch x dims[nLayers]. Runs `steps` steps, writes the loss of each step and
// returns the seconds spent in the steps.
double aixref_mlp_train_f32(const size_t* dims, size_t nLayers, size_t batch, float** weights, float** biases,
                            const float* x, const float* y, size_t steps, float lr, float* losses)
{
    using namespace aix;
    nn::Sequential model;
    std::vector<nn::Linear*> linears;
    for (size_t l = 0; l < nLayers; ++l)
    {
        auto lin = new nn::Linear(dims[l], dims[l + 1]);
        std::memcpy(lin->m_w.value().data(), weights[l], dims[l] * dims[l + 1] * sizeof(float));
        std::memcpy(lin->m_b.value().data(), biases[l], dims[l + 1] * sizeof(float));
        linears.push_back(lin);
        model.add(lin);
        if (l + 1 < nLayers) model.add(new nn::Tanh());
    }
    auto tx = Tensor(x, batch * dims[0], DataType::kFloat32, Shape{batch, dims[0]});
    auto ty = Tensor(y, batch * dims[nLayers], DataType::kFloat32, Shape{batch, dims[nLayers]});
    optim::Adam optimizer(model.parameters(), lr);
    nn::MSELoss lossFunc;
    auto t0 = std::chrono::steady_clock::now();
    for (size_t s = 0; s < steps; ++s)
    {
        auto pred = model.forward(tx);
        auto loss = lossFunc(pred, ty);
        optimizer.zeroGrad();
        loss.backward();
        optimizer.step();
        if (losses) losses[s] = loss.value().item<float>();
    }
    auto t1 = std::chrono::steady_clock::now();
    for (size_t l = 0; l < nLayers; ++l)
    {
        std::memcpy(weights[l], linears[l]->m_w.value().data(), dims[l] * dims[l + 1] * sizeof(float));
        std::memcpy(biases[l], linears[l]->m_b.value().data(), dims[l + 1] * sizeof(float));
    }
    return std::chrono::duration<double>(t1 - t0).count();
}

}   // extern "C"
