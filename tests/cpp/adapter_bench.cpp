// Timing of the real drop-in path: the UNMODIFIED AIX front end (aix::Tensor, autograd, nn::Sequential, optim::Adam) on
// aix::DeviceB200 with managed memory - the configuration a user of the reference gets when they select the new device.
// Built against the reference headers by oracle/build_ref.py (the binary lands in oracle/_ref); bench.py runs it and
// carries its JSON line as `extras.cpp_front_end`.
//   * chain:  z = (a*b + c) * sigmoid(a) - tanh(b) / (1 + exp(-c)); s = z.sum()  on [rows, 1024] f32
//   * mlp:    4 Linear 1024-4096-4096-4096-1024 with tanh, MSE, Adam(1e-3), batch 4096: forward + backward + step
// Device time by events on the device's stream around the timed steps; host time = wall time the front end needs to
// issue one step (the chain synchronises after every evaluation, as the reference's device benchmarks do; the training
// loop never does, like the reference's examples). All tensors are created, uploaded and prefetched before the timed region.
#include "aixDeviceB200.hpp"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

using namespace aix;
using Clock = std::chrono::steady_clock;

static double seconds(Clock::time_point a, Clock::time_point b) { return std::chrono::duration<double>(b - a).count(); }

struct Timed { double deviceMs, hostMs, opsPerStep, launchesPerStep; };

template <class Step>
static Timed timeSteps(DeviceB200& device, int warmup, int steps, Step&& step)
{
    for (int i = 0; i < warmup; ++i) step();
    device.synchronize();
    aixb200_event *e0 = nullptr, *e1 = nullptr;
    aixb200_event_create(device.handle(), &e0);
    aixb200_event_create(device.handle(), &e1);
    aixb200_stats s0{}, s1{};
    aixb200_get_stats(device.handle(), &s0);
    aixb200_event_record(device.handle(), e0);
    const auto t0 = Clock::now();
    for (int i = 0; i < steps; ++i) step();
    const auto t1 = Clock::now();
    aixb200_event_record(device.handle(), e1);
    float ms = 0;
    aixb200_event_elapsed_ms(device.handle(), e0, e1, &ms);
    device.synchronize();
    aixb200_get_stats(device.handle(), &s1);
    aixb200_event_destroy(device.handle(), e0);
    aixb200_event_destroy(device.handle(), e1);
    return {ms / steps, 1e3 * seconds(t0, t1) / steps, double(s1.ops_recorded - s0.ops_recorded) / steps,
            double(s1.total_kernel_launches - s0.total_kernel_launches) / steps};
}

int main(int argc, char** argv)
{
    const size_t chainRows = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : (size_t(1) << 16);      // x 1024 columns
    const size_t batch = argc > 2 ? std::strtoull(argv[2], nullptr, 10) : 4096;
    const int steps = argc > 3 ? std::atoi(argv[3]) : 10;
    DeviceB200 device(0);
    TensorOptions opt{ .m_device = &device };
    std::mt19937 gen(0);

    // ---- fused chain ------------------------------------------------------------------------------------------------
    Timed chain{};
    float chainSum = 0;
    {
        const size_t n = chainRows * 1024;
        std::uniform_real_distribution<float> dist(-1.f, 1.f);
        std::vector<float> host(n);
        Tensor t[3];
        for (auto& x : t)
        {
            for (auto& v : host) v = dist(gen);
            x = Tensor(host.data(), n, DataType::kFloat32, Shape{chainRows, 1024}, opt);
        }
        device.synchronize();
        Tensor s;
        chain = timeSteps(device, 3, steps, [&]
        {
            auto z = (t[0] * t[1] + t[2]) * (1 / (1 + (-t[0]).exp())) - t[1].tanh() / (1 + (-t[2]).exp());
            s = z.sum();
            device.synchronize();          // one evaluation per synchronisation, as the reference's own benchmarks run (Bench/Device.cpp)
        });
        chainSum = s.value().item<float>();
    }
    device.emptyCache();

    // ---- MLP training step ---------------------------------------------------------------------------------------------
    Timed mlp{};
    float firstLoss = 0, lastLoss = 0;
    const size_t dims[5] = {1024, 4096, 4096, 4096, 1024};
    {
        nn::Sequential model;
        for (int i = 0; i < 4; ++i)
        {
            auto layer = new nn::Linear(dims[i], dims[i + 1]);
            const float bound = std::sqrt(6.0f / float(dims[i] + dims[i + 1]));        // Xavier-uniform, written in place on the host
            std::uniform_real_distribution<float> dist(-bound, bound);
            float* w = layer->m_w.value().data<float>();
            for (size_t k = 0; k < dims[i] * dims[i + 1]; ++k) w[k] = dist(gen);
            std::memset(layer->m_b.value().data<float>(), 0, dims[i + 1] * sizeof(float));
            model.add(layer);
            if (i < 3) model.add(new nn::Tanh());
        }
        model.to(&device);
        std::normal_distribution<float> normal(0.f, 1.f);
        std::vector<float> x(batch * dims[0]), y(batch * dims[4]);
        for (auto& v : x) v = normal(gen);
        for (auto& v : y) v = normal(gen);
        auto inputs = Tensor(x.data(), x.size(), DataType::kFloat32, Shape{batch, dims[0]}, opt);
        auto targets = Tensor(y.data(), y.size(), DataType::kFloat32, Shape{batch, dims[4]}, opt);
        optim::Adam optimizer(model.parameters(), 1e-3f);            // created after the parameters live on the device
        nn::MSELoss lossFunc;
        Tensor loss;
        auto step = [&]
        {
            auto pred = model.forward(inputs);
            loss = lossFunc(pred, targets);
            optimizer.zeroGrad();
            loss.backward();
            optimizer.step();
        };
        step();
        device.synchronize();
        firstLoss = loss.value().item<float>();
        mlp = timeSteps(device, 2, steps, step);
        lastLoss = loss.value().item<float>();
    }
    const double flops = 2.0 * batch * (1024.0 * 4096 + 4096.0 * 4096 * 2 + 4096.0 * 1024) * 3 - 2.0 * batch * 1024.0 * 4096;
    std::printf("{\"device\": \"%s\", \"memory\": \"managed\", \"steps\": %d, "
                "\"chain\": {\"elements\": %zu, \"device_ms_per_step\": %.5f, \"host_ms_per_step\": %.5f, \"GB/s\": %.1f, \"device_calls_recorded_per_step\": %.1f, "
                "\"kernel_launches_per_step\": %.1f, \"sum\": %.6g}, "
                "\"mlp\": {\"batch\": %zu, \"device_ms_per_step\": %.5f, \"host_ms_per_step\": %.5f, \"gemm_TFLOP/s\": %.1f, \"device_calls_recorded_per_step\": %.1f, "
                "\"kernel_launches_per_step\": %.1f, \"host_us_per_recorded_call\": %.2f, \"loss_first\": %.6g, \"loss_last\": %.6g}}\n",
                device.name().c_str(), steps, chainRows * 1024, chain.deviceMs, chain.hostMs, 16.0 * chainRows * 1024 / (chain.deviceMs * 1e-3) / 1e9,
                chain.opsPerStep, chain.launchesPerStep, chainSum, batch, mlp.deviceMs, mlp.hostMs, flops / (mlp.deviceMs * 1e-3) / 1e12, mlp.opsPerStep,
                mlp.launchesPerStep, 1e3 * mlp.hostMs / std::max(1.0, mlp.opsPerStep), firstLoss, lastLoss);
    return (std::isfinite(lastLoss) && lastLoss < firstLoss) ? 0 : 1;
}
