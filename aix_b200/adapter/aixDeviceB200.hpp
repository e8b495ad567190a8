// aix::DeviceB200 - the reference-side binding of the B200 device.
//
// A header-only aix::Device subclass (Targets/AIXLib/aixDevice.hpp:30-84) that forwards every virtual to the C ABI of
// libaixb200.so (include/aixb200.h). Drop it next to the AIX headers, link libaixb200.so, and use it exactly like the
// Metal device:   auto device = aix::b200::createDevice(0);   model.to(device);   ...   device->synchronize();
// The device is created with managed_memory = 1, because the AIX core dereferences tensor storage on the host
// (TensorValue::item, getValueAt, nn::save/load - aixCore.hpp:435-440, 491-499); call synchronize() before doing so,
// as with the Metal device.
//
// Status codes of the C ABI become the exceptions the reference's devices throw: AIXB200_ERR_INVALID ->
// std::invalid_argument, everything else -> std::runtime_error.
#pragma once

#include "aix.hpp"
#include "aixb200.h"

#include <memory>
#include <stdexcept>
#include <string>

namespace aix
{

// Value outside the reference's enum {kCPU, kGPU_METAL} (aixDeviceType.hpp:15-19).
constexpr DeviceType kGPU_B200 = static_cast<DeviceType>(2);

class DeviceB200 : public Device
{
public:
    explicit DeviceB200(size_t deviceIndex = 0)
    {
        aixb200_config cfg;
        aixb200_default_config(&cfg);
        cfg.ordinal = static_cast<int32_t>(deviceIndex);
        cfg.managed_memory = 1;
        if (int status = aixb200_create_with_config(&cfg, &m_dev); status != AIXB200_OK)
            throw std::runtime_error(std::string("DeviceB200: ") + aixb200_last_error(nullptr));
    }
    ~DeviceB200() override { aixb200_destroy(m_dev); }
    DeviceB200(const DeviceB200&) = delete;
    DeviceB200& operator=(const DeviceB200&) = delete;

    DeviceType type() const override { return kGPU_B200; }
    std::string name() const override { return aixb200_name(m_dev); }

    void* allocate(size_t size) override { void* p = nullptr; check(aixb200_allocate(m_dev, size, &p)); return p; }
    void* allocate(size_t size, DataType dtype) override
    {
        void* p = nullptr;
        check(aixb200_allocate_typed(m_dev, size, static_cast<uint32_t>(dtype), &p));
        return p;
    }
    void deallocate(void* memory) override { check(aixb200_deallocate(m_dev, memory)); }

    void add(const DeviceTensorParams& a1, const DeviceTensorParams& a2, const DeviceTensorParams& r) override { T a(a1), b(a2), c(r); check(aixb200_add(m_dev, a, b, c)); }
    void sub(const DeviceTensorParams& a1, const DeviceTensorParams& a2, const DeviceTensorParams& r) override { T a(a1), b(a2), c(r); check(aixb200_sub(m_dev, a, b, c)); }
    void mul(const DeviceTensorParams& a1, const DeviceTensorParams& a2, const DeviceTensorParams& r) override { T a(a1), b(a2), c(r); check(aixb200_mul(m_dev, a, b, c)); }
    void div(const DeviceTensorParams& a1, const DeviceTensorParams& a2, const DeviceTensorParams& r) override { T a(a1), b(a2), c(r); check(aixb200_div(m_dev, a, b, c)); }
    void unary(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_unary(m_dev, a, c)); }
    void fill(const void* scalar, DataType scalarDType, const DeviceTensorParams& r) override { T c(r); check(aixb200_fill(m_dev, scalar, static_cast<uint32_t>(scalarDType), c)); }
    void fillMin(const DeviceTensorParams& r) override { T c(r); check(aixb200_fill_min(m_dev, c)); }
    void sum(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_sum(m_dev, a, c)); }
    void sqrt(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_sqrt(m_dev, a, c)); }
    void sin(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_sin(m_dev, a, c)); }
    void cos(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_cos(m_dev, a, c)); }
    void tanh(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_tanh(m_dev, a, c)); }
    void log(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_log(m_dev, a, c)); }
    void exp(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_exp(m_dev, a, c)); }
    void pow(const DeviceTensorParams& a1, const DeviceTensorParams& e, const DeviceTensorParams& r) override { T a(a1), b(e), c(r); check(aixb200_pow(m_dev, a, b, c)); }
    void max(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_max(m_dev, a, c)); }
    void argmax(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_argmax(m_dev, a, c)); }
    void argmaxIndices(const DeviceTensorParams& a1, const DeviceTensorParams& r) override { T a(a1), c(r); check(aixb200_argmax_indices(m_dev, a, c)); }
    void matmul(const DeviceTensorParams& a1, const DeviceTensorParams& a2, const DeviceTensorParams& r) override { T a(a1), b(a2), c(r); check(aixb200_matmul(m_dev, a, b, c)); }
    void transpose(const DeviceTensorParams& a1, const DeviceTensorParams& r, size_t dim0, size_t dim1) override { T a(a1), c(r); check(aixb200_transpose(m_dev, a, c, dim0, dim1)); }
    void copy(const void* src, DataType srcDType, void* dst, DataType dstDType, size_t size) override
    { check(aixb200_copy(m_dev, src, static_cast<uint32_t>(srcDType), dst, static_cast<uint32_t>(dstDType), size)); }
    void copyImmediate(const void* src, DataType srcDType, void* dst, DataType dstDType, size_t size) override
    { check(aixb200_copy_immediate(m_dev, src, static_cast<uint32_t>(srcDType), dst, static_cast<uint32_t>(dstDType), size)); }
    void contiguous(const DeviceTensorParams& s, const DeviceTensorParams& d) override { T a(s), c(d); check(aixb200_contiguous(m_dev, a, c)); }
    void reduceTo(const DeviceTensorParams& s, const DeviceTensorParams& d) override { T a(s), c(d); check(aixb200_reduce_to(m_dev, a, c)); }
    void maxTo(const DeviceTensorParams& s, const DeviceTensorParams& d) override { T a(s), c(d); check(aixb200_max_to(m_dev, a, c)); }
    void argmaxTo(const DeviceTensorParams& s, const DeviceTensorParams& d, size_t dim) override { T a(s), c(d); check(aixb200_argmax_to(m_dev, a, c, dim)); }
    void argmaxIndicesTo(const DeviceTensorParams& s, const DeviceTensorParams& d, size_t dim) override { T a(s), c(d); check(aixb200_argmax_indices_to(m_dev, a, c, dim)); }
    void sliceSet(const DeviceTensorParams& s, const DeviceTensorParams& d, size_t dim, size_t start, size_t end, size_t step) override
    { T a(s), c(d); check(aixb200_slice_set(m_dev, a, c, dim, start, end, step)); }
    void tril(const DeviceTensorParams& s, const DeviceTensorParams& d, ssize_t diagonal) override { T a(s), c(d); check(aixb200_tril(m_dev, a, c, diagonal)); }
    void triu(const DeviceTensorParams& s, const DeviceTensorParams& d, ssize_t diagonal) override { T a(s), c(d); check(aixb200_triu(m_dev, a, c, diagonal)); }
    void indexSelect(const DeviceTensorParams& s, const DeviceTensorParams& d, const DeviceTensorParams& indices, size_t dim) override
    { T a(s), c(d), i(indices); check(aixb200_index_select(m_dev, a, c, i, dim)); }
    void indexAdd(const DeviceTensorParams& s, const DeviceTensorParams& d, const DeviceTensorParams& indices, size_t dim) override
    { T a(s), c(d), i(indices); check(aixb200_index_add(m_dev, a, c, i, dim)); }
    void emptyCache() override { check(aixb200_empty_cache(m_dev)); }
    void synchronize() override { check(aixb200_synchronize(m_dev)); }

    aixb200_device* handle() const { return m_dev; }

private:
    // DeviceTensorParams -> POD descriptor; converts implicitly to the pointer the C ABI takes.
    struct T
    {
        aixb200_tensor t{};
        explicit T(const DeviceTensorParams& p)
        {
            if (p.shape.size() > AIXB200_MAX_RANK) throw std::invalid_argument("DeviceB200: tensor rank above AIXB200_MAX_RANK.");
            t.data = p.data;
            t.offset = p.offset;
            t.size = p.size;
            t.dtype = static_cast<uint32_t>(p.dtype);
            t.rank = static_cast<uint32_t>(p.shape.size());
            for (size_t i = 0; i < p.shape.size(); ++i) { t.shape[i] = p.shape[i]; t.strides[i] = p.strides[i]; }
        }
        operator const aixb200_tensor*() const { return &t; }
    };

    void check(int status) const
    {
        if (status == AIXB200_OK) return;
        const std::string message = aixb200_last_error(m_dev);
        if (status == AIXB200_ERR_INVALID) throw std::invalid_argument(message);
        throw std::runtime_error(message);
    }

    aixb200_device* m_dev{nullptr};
};

namespace b200
{
// Counterpart of aix::createDevice (aixDevices.cpp:24-43) for this device type.
inline std::unique_ptr<Device> createDevice(size_t deviceIndex = 0) { return std::make_unique<DeviceB200>(deviceIndex); }
}   // namespace b200

}   // namespace aix
