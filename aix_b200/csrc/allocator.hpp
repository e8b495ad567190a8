// Caching device allocator.
//
// Plays the role of the reference's MetalAllocator + MTLBufferCache (aixDeviceMetalCache.hpp:28-330): requests are
// rounded to size classes, freed blocks are parked in a size-ordered cache and handed out again without touching
// the CUDA allocator, and the cache is trimmed when it grows past a limit or when CUDA runs out of memory
// (retry-after-trim like aixDeviceMetal.cpp:1433-1475).
//
// Lifetime rule: everything the device does runs on one in-order stream, so a block may be reused as soon as the
// work that referenced it has been *enqueued*. The device therefore hands blocks back (release()) only after the
// recorded ops that mention them were emitted; the allocator itself never waits on the GPU except inside trim().
#pragma once

#include "common.hpp"

#include <functional>
#include <map>
#include <algorithm>

namespace aixb200
{

struct RawMemoryOps
{
    // Returns nullptr on out-of-memory; throws on any other failure.
    std::function<void*(size_t bytes)> allocate;
    std::function<void(void*)> free;
};

class CachingAllocator
{
public:
    CachingAllocator(RawMemoryOps raw, uint64_t cacheLimitBytes) : m_raw(std::move(raw)), m_cacheLimit(cacheLimitBytes) {}
    ~CachingAllocator() { releaseAll(); }

    static size_t roundSize(size_t bytes)
    {
        if (bytes == 0) bytes = 1;
        if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);                   // 512 B classes up to 1 MiB
        return (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);              // 2 MiB pages above
    }

    void* allocate(size_t bytes)
    {
        const size_t rounded = roundSize(bytes);
        // Best fit, but never waste more than a quarter of the request.
        auto it = m_cache.lower_bound(rounded);
        if (it != m_cache.end() && it->first <= rounded + rounded / 4)
        {
            void* p = it->second;
            m_cached -= it->first;
            m_live.emplace(p, it->first);
            m_inUse += it->first;
            m_cache.erase(it);
            ++m_cacheHits;
            return p;
        }
        void* p = m_raw.allocate(rounded);
        if (!p)
        {
            trim(0);
            p = m_raw.allocate(rounded);
            if (!p) failRuntime("device allocation of " + std::to_string(rounded) + " bytes failed after emptying the cache");
        }
        ++m_rawAllocs;
        m_reserved += rounded;
        m_live.emplace(p, rounded);
        m_inUse += rounded;
        return p;
    }

    // True if p is the base address of a live block.
    bool owns(const void* p) const { return m_live.count(const_cast<void*>(p)) != 0; }

    // Finds the live block that contains p; returns its base (nullptr if p is foreign) and its size.
    void* findBlock(const void* p, size_t* size = nullptr) const
    {
        auto it = m_live.upper_bound(const_cast<void*>(p));
        if (it == m_live.begin()) return nullptr;
        --it;
        auto base = static_cast<const char*>(it->first);
        if (static_cast<const char*>(p) >= base + it->second) return nullptr;
        if (size) *size = it->second;
        return it->first;
    }

    size_t blockSize(const void* p) const
    {
        auto it = m_live.find(const_cast<void*>(p));
        return it == m_live.end() ? 0 : it->second;
    }

    // Parks a live block in the cache.
    void release(void* p)
    {
        auto it = m_live.find(p);
        if (it == m_live.end()) failInvalid("deallocate: pointer was not allocated by this device");
        const size_t size = it->second;
        m_live.erase(it);
        m_inUse -= size;
        m_cache.emplace(size, p);
        m_cached += size;
        if (m_cached > m_cacheLimit) trim(m_cacheLimit / 2);
    }

    // Frees cached blocks, largest first, until at most `keepBytes` stay cached.
    void trim(uint64_t keepBytes)
    {
        while (m_cached > keepBytes && !m_cache.empty())
        {
            auto it = std::prev(m_cache.end());
            m_raw.free(it->second);
            m_cached -= it->first;
            m_reserved -= it->first;
            m_cache.erase(it);
        }
    }

    void releaseAll()
    {
        trim(0);
        for (auto& [p, size] : m_live) { m_raw.free(p); m_reserved -= size; }
        m_live.clear();
        m_inUse = 0;
    }

    uint64_t bytesInUse() const { return m_inUse; }
    uint64_t bytesCached() const { return m_cached; }
    uint64_t bytesReserved() const { return m_reserved; }
    uint64_t rawAllocations() const { return m_rawAllocs; }
    uint64_t cacheHits() const { return m_cacheHits; }

private:
    RawMemoryOps m_raw;
    uint64_t m_cacheLimit;
    std::multimap<size_t, void*> m_cache;              // idle blocks by size
    std::map<void*, size_t> m_live;                    // blocks handed out, ordered by address
    uint64_t m_inUse = 0, m_cached = 0, m_reserved = 0, m_rawAllocs = 0, m_cacheHits = 0;
};

}   // namespace aixb200
