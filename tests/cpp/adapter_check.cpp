// Drop-in check: the UNMODIFIED AIX front end (aix::Tensor, autograd, nn, optim) running on aix::DeviceB200, next to
// the same program on aix::DeviceCPU. Built against the reference headers by oracle/build_ref.py (test infrastructure;
// the binary lands in oracle/_ref) and run on a GPU by tests/test_gpu_adapter.py.
// Prints one "name: ok|FAIL detail" line per check and exits non-zero on any failure.
#include "aixDeviceB200.hpp"

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

using namespace aix;

static int failures = 0;
static void report(const char* name, bool ok, double detail)
{
    std::printf("%s: %s (%.3g)\n", name, ok ? "ok" : "FAIL", detail);
    if (!ok) ++failures;
}

static std::vector<float> uniform(size_t n, unsigned seed, float lo = -1.f, float hi = 1.f)
{
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> dist(lo, hi);
    std::vector<float> v(n);
    for (auto& x : v) x = dist(gen);
    return v;
}

static double maxRelDiff(const TensorValue& a, const TensorValue& b)
{
    double worst = 0;
    for (size_t i = 0; i < a.size(); ++i)
    {
        double x = a.data<float>()[i], y = b.data<float>()[i];
        worst = std::max(worst, std::fabs(x - y) / std::max(1.0, std::fabs(y)));
    }
    return worst;
}

// z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c)); s = z.sum()
static std::pair<Tensor, Tensor> chain(Device* device, const std::vector<float>& a, const std::vector<float>& b, const std::vector<float>& c, size_t rows, size_t cols)
{
    TensorOptions opt{ .m_device = device };
    Shape shape{rows, cols};
    auto ta = Tensor(a.data(), a.size(), DataType::kFloat32, shape, opt);
    auto tb = Tensor(b.data(), b.size(), DataType::kFloat32, shape, opt);
    auto tc = Tensor(c.data(), c.size(), DataType::kFloat32, shape, opt);
    auto z = (ta * tb + tc) * (1 / (1 + (-ta).exp())) - tb.tanh() / (1 + (-tc).exp());
    auto s = z.sum();
    device->synchronize();
    return {z, s};
}

static std::vector<float> trainXor(Device* device, size_t epochs, float* finalLoss)
{
    // The README's XOR example: 2 -> 8 -> 1 with tanh, Adam, MSE, no synchronize inside the loop.
    std::vector<float> w1 = uniform(2 * 8, 1), b1 = uniform(8, 2), w2 = uniform(8, 3), b2 = uniform(1, 4);
    nn::Sequential model;
    auto l1 = new nn::Linear(2, 8);
    auto l2 = new nn::Linear(8, 1);
    std::memcpy(l1->m_w.value().data(), w1.data(), w1.size() * 4);
    std::memcpy(l1->m_b.value().data(), b1.data(), b1.size() * 4);
    std::memcpy(l2->m_w.value().data(), w2.data(), w2.size() * 4);
    std::memcpy(l2->m_b.value().data(), b2.data(), b2.size() * 4);
    model.add(l1);
    model.add(new nn::Tanh());
    model.add(l2);
    model.to(device);
    TensorOptions opt{ .m_device = device };
    auto inputs = tensor({0.f, 0.f, 0.f, 1.f, 1.f, 0.f, 1.f, 1.f}, Shape{4, 2}, opt);
    auto targets = tensor({0.f, 1.f, 1.f, 0.f}, Shape{4, 1}, opt);
    optim::Adam optimizer(model.parameters(), 0.05f);
    nn::MSELoss lossFunc;
    Tensor loss;
    for (size_t e = 0; e < epochs; ++e)
    {
        auto pred = model.forward(inputs);
        loss = lossFunc(pred, targets);
        optimizer.zeroGrad();
        loss.backward();
        optimizer.step();
    }
    device->synchronize();
    *finalLoss = loss.value().item<float>();
    auto pred = model.forward(inputs);
    device->synchronize();
    std::vector<float> out(4);
    for (size_t i = 0; i < 4; ++i) out[i] = pred.value().data<float>()[i];
    return out;
}

int main()
{
    auto gpu = b200::createDevice(0);
    DeviceCPU cpu;
    std::printf("device: %s\n", gpu->name().c_str());

    {   // fused chain at config-0 size
        const size_t rows = 1024, cols = 1024;
        auto a = uniform(rows * cols, 0), b = uniform(rows * cols, 1), c = uniform(rows * cols, 2);
        auto [zg, sg] = chain(gpu.get(), a, b, c, rows, cols);
        auto [zc, sc] = chain(&cpu, a, b, c, rows, cols);
        report("chain z", maxRelDiff(zg.value(), zc.value()) <= 1e-5, maxRelDiff(zg.value(), zc.value()));
        double exact = 0, absSum = 0;
        for (size_t i = 0; i < zc.value().size(); ++i) { exact += zc.value().data<float>()[i]; absSum += std::fabs(zc.value().data<float>()[i]); }
        report("chain sum", std::fabs(sg.value().item<float>() - exact) <= 1e-5 * std::max(1.0, std::fabs(exact)), sg.value().item<float>() - exact);
    }
    {   // matmul forward + autograd backward with transposed views
        const size_t n = 192;
        auto a = uniform(n * n, 5, -0.05f, 0.05f), b = uniform(n * n, 6, -0.05f, 0.05f);
        Tensor grads[2][2];
        Tensor outs[2];
        Device* devices[2] = {gpu.get(), &cpu};
        for (int d = 0; d < 2; ++d)
        {
            TensorOptions opt{ .m_requireGrad = true, .m_device = devices[d] };
            auto ta = Tensor(a.data(), a.size(), DataType::kFloat32, Shape{n, n}, opt);
            auto tb = Tensor(b.data(), b.size(), DataType::kFloat32, Shape{n, n}, opt);
            auto c = matmul(ta, tb);
            c.backward(Tensor(1.0f, Shape{n, n}, TensorOptions{ .m_device = devices[d] }));   // upstream gradient of ones
            devices[d]->synchronize();
            outs[d] = c; grads[d][0] = ta; grads[d][1] = tb;
        }
        auto normwise = [](const TensorValue& x, const TensorValue& y)
        {
            double worst = 0, scale = 0;
            for (size_t i = 0; i < x.size(); ++i) { worst = std::max(worst, (double)std::fabs(x.data<float>()[i] - y.data<float>()[i])); scale = std::max(scale, (double)std::fabs(y.data<float>()[i])); }
            return worst / scale;
        };
        report("matmul C", normwise(outs[0].value(), outs[1].value()) <= 1e-5, normwise(outs[0].value(), outs[1].value()));
        report("matmul dA", normwise(grads[0][0].grad(), grads[1][0].grad()) <= 1e-5, normwise(grads[0][0].grad(), grads[1][0].grad()));
        report("matmul dB", normwise(grads[0][1].grad(), grads[1][1].grad()) <= 1e-5, normwise(grads[0][1].grad(), grads[1][1].grad()));
    }
    {   // training loop without synchronize (Tests/DeviceTests.cpp:3503-3552)
        float lossGpu = 0, lossCpu = 0;
        auto pg = trainXor(gpu.get(), 300, &lossGpu);
        auto pc = trainXor(&cpu, 300, &lossCpu);
        double worst = 0;
        for (size_t i = 0; i < 4; ++i) worst = std::max(worst, (double)std::fabs(pg[i] - pc[i]));
        report("xor predictions", worst <= 2e-3, worst);
        report("xor converged", lossGpu <= 1e-2, lossGpu);
    }
    std::printf("%s\n", failures ? "FAILED" : "ALL OK");
    return failures ? 1 : 0;
}
